// TEST INFRASTRUCTURE. C entry points onto the REFERENCE's own four operations (reference src/upstride.hpp:18-86),
// compiled from the reference's sources where they lie, with `dnnl_stub/dnnl.hpp` standing in for oneDNN (every scalar
// convolution / matrix product a direct double-accumulating loop). What runs is the reference's algebra composition:
// UpstrideConv2DFunctor / UpstrideConv2DGradFunctor (src/conv2d.hpp), UpstrideDenseFunctor / GradFunctor
// (src/dense.hpp), its sign tables (src/algebras.cc), its quaternion lane arithmetic (src/backend/onednn/tensor.cc)
// and its descriptor geometry (src/backend/conv2d_descriptor.hpp). Used only to check the oracle and to generate the
// golden vectors under tests/golden/; never linked into or called by the product.
#include <cstdlib>
#include <exception>
#include <cstdio>

#include "upstride.hpp"

using namespace upstride;

namespace {

struct Engine {
    onednn::Context* context;
    device::CPU* device;
};

// One context + device per formulation: the reference reads UPSTRIDE_MEMORY_OPTIMIZED when a Context is constructed
// (src/backend/backend.cc:45-47); 0 selects the factorised 8-product quaternion path, 1 the 16-product one.
Engine& engine_for(int memory_optimized) {
    static Engine engines[2] = {{nullptr, nullptr}, {nullptr, nullptr}};
    Engine& e = engines[memory_optimized ? 1 : 0];
    if (!e.context) {
        setenv("UPSTRIDE_MEMORY_OPTIMIZED", memory_optimized ? "1" : "0", 1);
        e.context = new onednn::Context();
        e.device = new device::CPU(*e.context);
    }
    return e;
}

IntTuple tuple_of(const int* v, int n) { return IntTuple(v, v + n); }

template <typename F>
int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::exception& ex) {
        std::fprintf(stderr, "reference raised: %s\n", ex.what());
        return 1;
    }
}

}  // namespace

extern "C" {

// Shapes are given as int arrays with their rank. padding_preset: 0 SAME, 1 VALID, 2 EXPLICIT (then `pad` holds the
// reference's explicit padding tuple). algebra / data_format / filter_layout are the reference's enum values.
int ref_conv2d_fwd(int memory_optimized, const float* x, const int* xs, int xr, const float* w, const int* ws, int wr, const float* bias,
                   const int* bs, int br, float* y, const int* ys, int yr, int stride_a, int stride_b, int dil_a, int dil_b,
                   int padding_preset, const int* pad, int n_pad, int groups, int algebra, int data_format, int filter_layout,
                   int real_input) {
    return guarded([&] {
        Engine& e = engine_for(memory_optimized);
        const Shape xshape(xr, xs), wshape(wr, ws), yshape(yr, ys);
        Conv2DFwdDescriptor desc(xshape, wshape, IntPair(stride_a, stride_b), IntPair(dil_a, dil_b), (Padding)padding_preset, tuple_of(pad, n_pad),
                                 groups, (Algebra)algebra, (DataFormat)data_format, (FilterLayout)filter_layout, bias != nullptr, real_input != 0);
        const Tensor<device::CPU, const float> tx(*e.device, xshape, x), tw(*e.device, wshape, w);
        Tensor<device::CPU, float> ty(*e.device, yshape, y);
        if (bias) {
            const Shape bshape(br, bs);
            const Tensor<device::CPU, const float> tb(*e.device, bshape, bias);
            conv2DFwd<device::CPU, float>(*e.device, *e.device, tx, tw, &tb, ty, desc);
        } else {
            conv2DFwd<device::CPU, float>(*e.device, *e.device, tx, tw, nullptr, ty, desc);
        }
    });
}

int ref_conv2d_bwd(int memory_optimized, const float* x, const int* xs, int xr, const float* w, const int* ws, int wr, const float* dy,
                   const int* ys, int yr, float* dw, float* dx, int stride_a, int stride_b, int dil_a, int dil_b, int padding_preset,
                   const int* pad, int n_pad, int groups, int algebra, int data_format, int filter_layout, int need_dx, int real_input) {
    return guarded([&] {
        Engine& e = engine_for(memory_optimized);
        const Shape xshape(xr, xs), wshape(wr, ws), yshape(yr, ys);
        Conv2DBwdDescriptor desc(xshape, wshape, IntPair(stride_a, stride_b), IntPair(dil_a, dil_b), (Padding)padding_preset, tuple_of(pad, n_pad),
                                 groups, (Algebra)algebra, (DataFormat)data_format, (FilterLayout)filter_layout, need_dx != 0, real_input != 0);
        const Tensor<device::CPU, const float> tx(*e.device, xshape, x), tw(*e.device, wshape, w), tdy(*e.device, yshape, dy);
        Tensor<device::CPU, float> tdw(*e.device, wshape, dw), tdx(*e.device, xshape, dx);
        conv2DBwd<device::CPU, float>(*e.device, *e.device, tx, tw, tdy, tdw, tdx, desc);
    });
}

int ref_dense_fwd(int memory_optimized, const float* x, const int* xs, const float* w, const int* ws, int wr, const float* bias, const int* bs,
                  int br, float* y, const int* ys, int algebra, int filter_layout) {
    return guarded([&] {
        Engine& e = engine_for(memory_optimized);
        const Shape xshape(2, xs), wshape(wr, ws), yshape(2, ys);
        DenseFwdDescriptor desc(xshape, wshape, (Algebra)algebra, (FilterLayout)filter_layout, bias != nullptr);
        const Tensor<device::CPU, const float> tx(*e.device, xshape, x), tw(*e.device, wshape, w);
        Tensor<device::CPU, float> ty(*e.device, yshape, y);
        if (bias) {
            const Shape bshape(br, bs);
            const Tensor<device::CPU, const float> tb(*e.device, bshape, bias);
            denseFwd<device::CPU, float>(*e.device, *e.device, tx, tw, &tb, ty, desc);
        } else {
            denseFwd<device::CPU, float>(*e.device, *e.device, tx, tw, nullptr, ty, desc);
        }
    });
}

// dw is written in the shape the reference gives the filter gradient (the filter's own shape object; the scalar
// backend fills it input-major whatever the layout).
int ref_dense_bwd(int memory_optimized, const float* x, const int* xs, const float* w, const int* ws, int wr, const float* dy, const int* ys,
                  float* dw, float* dx, int algebra, int filter_layout, int need_dx) {
    return guarded([&] {
        Engine& e = engine_for(memory_optimized);
        const Shape xshape(2, xs), wshape(wr, ws), yshape(2, ys);
        DenseBwdDescriptor desc(xshape, wshape, (Algebra)algebra, (FilterLayout)filter_layout, need_dx != 0);
        const Tensor<device::CPU, const float> tx(*e.device, xshape, x), tw(*e.device, wshape, w), tdy(*e.device, yshape, dy);
        Tensor<device::CPU, float> tdw(*e.device, wshape, dw), tdx(*e.device, xshape, dx);
        denseBwd<device::CPU, float>(*e.device, *e.device, tx, tw, tdy, tdw, tdx, desc);
    });
}

}  // extern "C"

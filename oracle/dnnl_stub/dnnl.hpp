// TEST INFRASTRUCTURE. A stand-in for the part of the oneDNN C++ API (`dnnl.hpp`) that the reference's CPU backend calls
// (reference src/backend/onednn/{context,conv2d,dense}.hpp), written from the published API's names and argument
// meaning, with every primitive computed by direct loops that accumulate in double. It exists so that the
// reference's OWN sources -- its algebra composition (src/conv2d.hpp, src/dense.hpp, src/algebras.*), its lane
// arithmetic (src/backend/onednn/tensor.*) and its scalar-functor glue -- compile and run here without oneDNN; what
// they compute is then the reference's composition over exact scalar convolutions and matrix products.
//
// Only what the reference uses is here: f32 data; memory descriptors built from dims + a format tag (or `any`, which
// a primitive descriptor resolves to the plain nchw / oihw / goihw layout, so the reference's reorder glue runs when
// the caller's layout is another one); convolution forward / backward-weights / backward-data with strides, dilation
// (oneDNN convention: 0 = dense) and left padding; matmul with optional bias; reorder; engine and stream as tokens.
#pragma once
#include <cstddef>
#include <cstdint>
#include <functional>
#include <memory>
#include <stdexcept>
#include <unordered_map>
#include <vector>

#define DNNL_ARG_SRC 1
#define DNNL_ARG_FROM 1
#define DNNL_ARG_DST 17
#define DNNL_ARG_TO 17
#define DNNL_ARG_WEIGHTS 33
#define DNNL_ARG_BIAS 41
#define DNNL_ARG_DIFF_SRC 129
#define DNNL_ARG_DIFF_DST 145
#define DNNL_ARG_DIFF_WEIGHTS 161

namespace dnnl {

enum class prop_kind { forward_training, forward_inference, backward };
enum class algorithm { convolution_auto, convolution_direct };

struct engine {
    enum class kind { cpu };
    engine() {}
    engine(kind, size_t) {}
};

struct stream {
    stream() {}
    explicit stream(const engine&) {}
    void wait() {}
};

struct memory {
    typedef int64_t dim;
    typedef std::vector<dim> dims;
    enum class data_type { f32 };
    enum class format_tag { undef, any, x, ab, ba, nc, cn, nchw, nhwc, oihw, ohwi, hwio, goihw, gohwi, hwigo };

    // Logical dims (activations n,c,h,w; filters o,i,h,w or g,o,i,h,w; matrices rows,cols) and element strides.
    struct desc {
        dims extent, stride;
        bool unresolved = false;   // built with format_tag::any
        desc() {}
        desc(const dims& d, data_type, format_tag tag) : extent(d), stride(d.size(), 0) {
            if (tag == format_tag::any) { unresolved = true; return; }
            set_strides(order_of(tag, d.size()));
        }
        // `order` lists the dims from outermost to innermost
        void set_strides(const std::vector<int>& order) {
            if (order.size() != extent.size()) throw std::invalid_argument("dnnl stub: tag does not match the number of dims");
            dim s = 1;
            for (int k = (int)order.size() - 1; k >= 0; --k) { stride[order[k]] = s; s *= extent[order[k]]; }
            unresolved = false;
        }
        static std::vector<int> order_of(format_tag tag, size_t n) {
            switch (tag) {
                case format_tag::x: return {0};
                case format_tag::ab: case format_tag::nc: return {0, 1};
                case format_tag::ba: case format_tag::cn: return {1, 0};
                case format_tag::nchw: case format_tag::oihw: return {0, 1, 2, 3};
                case format_tag::nhwc: case format_tag::ohwi: return {0, 2, 3, 1};
                case format_tag::hwio: return {2, 3, 1, 0};
                case format_tag::goihw: return {0, 1, 2, 3, 4};
                case format_tag::gohwi: return {0, 1, 3, 4, 2};
                case format_tag::hwigo: return {3, 4, 2, 0, 1};
                default: break;
            }
            (void)n;
            throw std::invalid_argument("dnnl stub: unsupported format tag");
        }
        // the plain layout a primitive descriptor picks for an `any` descriptor
        desc resolved() const {
            if (!unresolved) return *this;
            desc r = *this;
            std::vector<int> order(extent.size());
            for (size_t i = 0; i < order.size(); ++i) order[i] = (int)i;
            r.set_strides(order);
            return r;
        }
        desc permute_axes(const std::vector<int>& perm) const {
            desc r = *this;
            for (size_t i = 0; i < perm.size(); ++i) { r.extent[perm[i]] = extent[i]; r.stride[perm[i]] = stride[i]; }
            return r;
        }
        size_t numel() const { size_t n = 1; for (dim e : extent) n *= (size_t)e; return n; }
        size_t get_size() const { return numel() * sizeof(float); }
        bool operator==(const desc& o) const { return extent == o.extent && stride == o.stride && unresolved == o.unresolved; }
        bool operator!=(const desc& o) const { return !(*this == o); }
    };

    desc md;
    void* handle = nullptr;
    memory() {}
    memory(const desc& d, const engine&, void* h) : md(d), handle(h) {}
    const desc& get_desc() const { return md; }
    void* get_data_handle() const { return handle; }
    float* f32() const { return static_cast<float*>(handle); }
};

typedef std::unordered_map<int, memory> exec_args;

struct primitive {
    std::shared_ptr<std::function<void(const exec_args&)>> run;
    primitive() {}
    void execute(const stream&, const exec_args& args) const {
        if (!run) throw std::runtime_error("dnnl stub: executing an empty primitive");
        (*run)(args);
    }
};

namespace stub {

inline const memory& arg(const exec_args& args, int key) {
    auto it = args.find(key);
    if (it == args.end()) throw std::invalid_argument("dnnl stub: missing primitive argument");
    return it->second;
}

// A filter descriptor seen as (g, o, i, h, w) whatever its rank.
struct FilterView {
    memory::dim G, O, I, KH, KW, sg, so, si, sh, sw;
    explicit FilterView(const memory::desc& d) {
        const size_t b = d.extent.size() == 5 ? 1 : 0;
        G = b ? d.extent[0] : 1; sg = b ? d.stride[0] : 0;
        O = d.extent[b]; I = d.extent[b + 1]; KH = d.extent[b + 2]; KW = d.extent[b + 3];
        so = d.stride[b]; si = d.stride[b + 1]; sh = d.stride[b + 2]; sw = d.stride[b + 3];
    }
    size_t at(memory::dim g, memory::dim o, memory::dim i, memory::dim h, memory::dim w) const {
        return (size_t)(g * sg + o * so + i * si + h * sh + w * sw);
    }
};

struct ConvGeometry {
    memory::desc src, weights, bias, dst;
    bool with_bias = false;
    memory::dims strides, dilates, pad_l;
    size_t s_at(memory::dim n, memory::dim c, memory::dim h, memory::dim w) const {
        return (size_t)(n * src.stride[0] + c * src.stride[1] + h * src.stride[2] + w * src.stride[3]);
    }
    size_t d_at(memory::dim n, memory::dim c, memory::dim h, memory::dim w) const {
        return (size_t)(n * dst.stride[0] + c * dst.stride[1] + h * dst.stride[2] + w * dst.stride[3]);
    }
    void resolve() { src = src.resolved(); weights = weights.resolved(); dst = dst.resolved(); }
};

// which: 0 forward (dst from src, weights[, bias]); 1 backward-weights (weights from src, dst); 2 backward-data (src from dst, weights)
inline void convolution(const ConvGeometry& g, int which, float* src, float* wei, const float* bias, float* dst) {
    const FilterView f(g.weights);
    const memory::dim N = g.src.extent[0], H = g.src.extent[2], W = g.src.extent[3];
    const memory::dim OH = g.dst.extent[2], OW = g.dst.extent[3];
    const memory::dim sh = g.strides[0], sw = g.strides[1], dh = g.dilates[0] + 1, dw = g.dilates[1] + 1;
    const memory::dim ph = g.pad_l[0], pw = g.pad_l[1];
    if (g.src.extent[1] != f.G * f.I || g.dst.extent[1] != f.G * f.O) throw std::invalid_argument("dnnl stub: channel mismatch");
    if (which == 0) {
        for (memory::dim n = 0; n < N; ++n)
            for (memory::dim gr = 0; gr < f.G; ++gr)
                for (memory::dim o = 0; o < f.O; ++o)
                    for (memory::dim oh = 0; oh < OH; ++oh)
                        for (memory::dim ow = 0; ow < OW; ++ow) {
                            double acc = bias ? (double)bias[gr * f.O + o] : 0.0;
                            for (memory::dim i = 0; i < f.I; ++i)
                                for (memory::dim kh = 0; kh < f.KH; ++kh) {
                                    const memory::dim ih = oh * sh - ph + kh * dh;
                                    if (ih < 0 || ih >= H) continue;
                                    for (memory::dim kw = 0; kw < f.KW; ++kw) {
                                        const memory::dim iw = ow * sw - pw + kw * dw;
                                        if (iw < 0 || iw >= W) continue;
                                        acc += (double)src[g.s_at(n, gr * f.I + i, ih, iw)] * (double)wei[f.at(gr, o, i, kh, kw)];
                                    }
                                }
                            dst[g.d_at(n, gr * f.O + o, oh, ow)] = (float)acc;
                        }
    } else if (which == 1) {
        for (memory::dim gr = 0; gr < f.G; ++gr)
            for (memory::dim o = 0; o < f.O; ++o)
                for (memory::dim i = 0; i < f.I; ++i)
                    for (memory::dim kh = 0; kh < f.KH; ++kh)
                        for (memory::dim kw = 0; kw < f.KW; ++kw) {
                            double acc = 0.0;
                            for (memory::dim n = 0; n < N; ++n)
                                for (memory::dim oh = 0; oh < OH; ++oh) {
                                    const memory::dim ih = oh * sh - ph + kh * dh;
                                    if (ih < 0 || ih >= H) continue;
                                    for (memory::dim ow = 0; ow < OW; ++ow) {
                                        const memory::dim iw = ow * sw - pw + kw * dw;
                                        if (iw < 0 || iw >= W) continue;
                                        acc += (double)src[g.s_at(n, gr * f.I + i, ih, iw)] * (double)dst[g.d_at(n, gr * f.O + o, oh, ow)];
                                    }
                                }
                            wei[f.at(gr, o, i, kh, kw)] = (float)acc;
                        }
    } else {
        for (memory::dim n = 0; n < N; ++n)
            for (memory::dim gr = 0; gr < f.G; ++gr)
                for (memory::dim i = 0; i < f.I; ++i)
                    for (memory::dim ih = 0; ih < H; ++ih)
                        for (memory::dim iw = 0; iw < W; ++iw) {
                            double acc = 0.0;
                            for (memory::dim kh = 0; kh < f.KH; ++kh) {
                                const memory::dim th = ih + ph - kh * dh;
                                if (th < 0 || th % sh != 0 || th / sh >= OH) continue;
                                for (memory::dim kw = 0; kw < f.KW; ++kw) {
                                    const memory::dim tw = iw + pw - kw * dw;
                                    if (tw < 0 || tw % sw != 0 || tw / sw >= OW) continue;
                                    for (memory::dim o = 0; o < f.O; ++o)
                                        acc += (double)dst[g.d_at(n, gr * f.O + o, th / sh, tw / sw)] * (double)wei[f.at(gr, o, i, kh, kw)];
                                }
                            }
                            src[g.s_at(n, gr * f.I + i, ih, iw)] = (float)acc;
                        }
    }
}

inline void copy_strided(const memory& from, const memory& to) {
    const memory::desc &a = from.get_desc(), &b = to.get_desc();
    if (a.extent != b.extent) throw std::invalid_argument("dnnl stub: reorder between different dims");
    const size_t rank = a.extent.size(), total = a.numel();
    std::vector<memory::dim> idx(rank, 0);
    for (size_t e = 0; e < total; ++e) {
        size_t oa = 0, ob = 0;
        for (size_t k = 0; k < rank; ++k) { oa += (size_t)(idx[k] * a.stride[k]); ob += (size_t)(idx[k] * b.stride[k]); }
        to.f32()[ob] = from.f32()[oa];
        for (int k = (int)rank - 1; k >= 0; --k) {
            if (++idx[k] < a.extent[k]) break;
            idx[k] = 0;
        }
    }
}

}  // namespace stub

struct convolution_forward : public primitive {
    struct desc {
        stub::ConvGeometry g;
        desc(prop_kind, algorithm, const memory::desc& src, const memory::desc& weights, const memory::desc& bias, const memory::desc& dst,
             const memory::dims& strides, const memory::dims& dilates, const memory::dims& pad_l, const memory::dims&) {
            g.src = src; g.weights = weights; g.bias = bias; g.dst = dst; g.with_bias = true;
            g.strides = strides; g.dilates = dilates; g.pad_l = pad_l;
        }
        desc(prop_kind, algorithm, const memory::desc& src, const memory::desc& weights, const memory::desc& dst,
             const memory::dims& strides, const memory::dims& dilates, const memory::dims& pad_l, const memory::dims&) {
            g.src = src; g.weights = weights; g.dst = dst;
            g.strides = strides; g.dilates = dilates; g.pad_l = pad_l;
        }
    };
    struct primitive_desc {
        stub::ConvGeometry g;
        primitive_desc() {}
        primitive_desc(const desc& d, const engine&) : g(d.g) { g.resolve(); }
        memory::desc src_desc() const { return g.src; }
        memory::desc weights_desc() const { return g.weights; }
        memory::desc dst_desc() const { return g.dst; }
    };
    convolution_forward() {}
    explicit convolution_forward(const primitive_desc& pd) {
        const stub::ConvGeometry g = pd.g;
        run = std::make_shared<std::function<void(const exec_args&)>>([g](const exec_args& a) {
            stub::convolution(g, 0, stub::arg(a, DNNL_ARG_SRC).f32(), stub::arg(a, DNNL_ARG_WEIGHTS).f32(),
                              g.with_bias ? stub::arg(a, DNNL_ARG_BIAS).f32() : nullptr, stub::arg(a, DNNL_ARG_DST).f32());
        });
    }
};

struct convolution_backward_weights : public primitive {
    struct desc {
        stub::ConvGeometry g;
        desc(algorithm, const memory::desc& src, const memory::desc& diff_weights, const memory::desc& diff_dst,
             const memory::dims& strides, const memory::dims& dilates, const memory::dims& pad_l, const memory::dims&) {
            g.src = src; g.weights = diff_weights; g.dst = diff_dst;
            g.strides = strides; g.dilates = dilates; g.pad_l = pad_l;
        }
    };
    struct primitive_desc {
        stub::ConvGeometry g;
        primitive_desc(const desc& d, const engine&, const convolution_forward::primitive_desc&) : g(d.g) { g.resolve(); }
        memory::desc src_desc() const { return g.src; }
        memory::desc diff_weights_desc() const { return g.weights; }
        memory::desc diff_dst_desc() const { return g.dst; }
    };
    convolution_backward_weights() {}
    explicit convolution_backward_weights(const primitive_desc& pd) {
        const stub::ConvGeometry g = pd.g;
        run = std::make_shared<std::function<void(const exec_args&)>>([g](const exec_args& a) {
            stub::convolution(g, 1, stub::arg(a, DNNL_ARG_SRC).f32(), stub::arg(a, DNNL_ARG_DIFF_WEIGHTS).f32(), nullptr,
                              stub::arg(a, DNNL_ARG_DIFF_DST).f32());
        });
    }
};

struct convolution_backward_data : public primitive {
    struct desc {
        stub::ConvGeometry g;
        desc(algorithm, const memory::desc& diff_src, const memory::desc& weights, const memory::desc& diff_dst,
             const memory::dims& strides, const memory::dims& dilates, const memory::dims& pad_l, const memory::dims&) {
            g.src = diff_src; g.weights = weights; g.dst = diff_dst;
            g.strides = strides; g.dilates = dilates; g.pad_l = pad_l;
        }
    };
    struct primitive_desc {
        stub::ConvGeometry g;
        primitive_desc(const desc& d, const engine&, const convolution_forward::primitive_desc&) : g(d.g) { g.resolve(); }
        memory::desc diff_src_desc() const { return g.src; }
        memory::desc weights_desc() const { return g.weights; }
        memory::desc diff_dst_desc() const { return g.dst; }
    };
    convolution_backward_data() {}
    explicit convolution_backward_data(const primitive_desc& pd) {
        const stub::ConvGeometry g = pd.g;
        run = std::make_shared<std::function<void(const exec_args&)>>([g](const exec_args& a) {
            stub::convolution(g, 2, stub::arg(a, DNNL_ARG_DIFF_SRC).f32(), stub::arg(a, DNNL_ARG_WEIGHTS).f32(), nullptr,
                              stub::arg(a, DNNL_ARG_DIFF_DST).f32());
        });
    }
};

struct reorder : public primitive {
    struct primitive_desc {
        primitive_desc(const engine&, const memory::desc&, const engine&, const memory::desc&) {}
    };
    reorder() {}
    explicit reorder(const primitive_desc&) {
        run = std::make_shared<std::function<void(const exec_args&)>>(
            [](const exec_args& a) { stub::copy_strided(stub::arg(a, DNNL_ARG_FROM), stub::arg(a, DNNL_ARG_TO)); });
    }
};

// dst[m, n] = sum_k src[m, k] * weights[k, n] (+ bias[0, n]); every operand addressed through its strides
struct matmul : public primitive {
    struct desc {
        memory::desc src, weights, bias, dst;
        bool with_bias;
        desc(const memory::desc& s, const memory::desc& w, const memory::desc& b, const memory::desc& d) : src(s), weights(w), bias(b), dst(d), with_bias(true) {}
        desc(const memory::desc& s, const memory::desc& w, const memory::desc& d) : src(s), weights(w), dst(d), with_bias(false) {}
    };
    struct primitive_desc {
        desc d;
        primitive_desc(const desc& dd, const engine&) : d(dd) {}
    };
    matmul() {}
    explicit matmul(const primitive_desc& pd) {
        const desc d = pd.d;
        if (d.src.extent[1] != d.weights.extent[0] || d.dst.extent[0] != d.src.extent[0] || d.dst.extent[1] != d.weights.extent[1])
            throw std::invalid_argument("dnnl stub: matmul dims do not agree");
        run = std::make_shared<std::function<void(const exec_args&)>>([d](const exec_args& a) {
            const float* s = stub::arg(a, DNNL_ARG_SRC).f32();
            const float* w = stub::arg(a, DNNL_ARG_WEIGHTS).f32();
            const float* b = d.with_bias ? stub::arg(a, DNNL_ARG_BIAS).f32() : nullptr;
            float* o = stub::arg(a, DNNL_ARG_DST).f32();
            const memory::dim M = d.src.extent[0], K = d.src.extent[1], N = d.weights.extent[1];
            for (memory::dim m = 0; m < M; ++m)
                for (memory::dim n = 0; n < N; ++n) {
                    double acc = b ? (double)b[n * d.bias.stride[1]] : 0.0;
                    for (memory::dim k = 0; k < K; ++k)
                        acc += (double)s[m * d.src.stride[0] + k * d.src.stride[1]] * (double)w[k * d.weights.stride[0] + n * d.weights.stride[1]];
                    o[m * d.dst.stride[0] + n * d.dst.stride[1]] = (float)acc;
                }
        });
    }
};

}  // namespace dnnl

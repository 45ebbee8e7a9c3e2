// C ABI of the backend: argument validation, geometry, kernel-family selection and dispatch.
// Nothing here allocates device memory; scratch comes from the caller's workspace.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tensor_path.cuh"
#include "umma.cuh"

namespace pcb {
int g_sm_margin = 0;         // SMs the persistent kernels leave free (pcb_set_sm_margin)

static thread_local char g_error[512] = {0};

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

namespace {

constexpr long long MAX_NUMEL = 2147483647LL;   // tensor offsets are 32-bit element indices inside kernels

int out_size(int in, int k, int dil, int stride, int before, int after) {
    const int eff = (k - 1) * dil + 1;
    return (in + before + after - eff + stride) / stride;
}

// Validates a convolution descriptor and fills the kernel geometry.
int conv_geom(const pcb_conv2d_desc* d, Geom& g) {
    if (!d) { set_error("null descriptor"); return PCB_ERR_INVALID_ARGUMENT; }
    if (d->dtype < PCB_F32 || d->dtype > PCB_BF16) { set_error("unknown dtype %d", d->dtype); return PCB_ERR_INVALID_ARGUMENT; }
    if (d->n < 0 || d->ci <= 0 || d->co <= 0 || d->h <= 0 || d->w <= 0 || d->kh <= 0 || d->kw <= 0 || d->stride_h <= 0 ||
        d->stride_w <= 0 || d->pad_top < 0 || d->pad_left < 0 || d->pad_bottom < 0 || d->pad_right < 0) {
        set_error("invalid convolution geometry");
        return PCB_ERR_INVALID_ARGUMENT;
    }
    if (d->groups < 1 || d->co % d->groups != 0) { set_error("invalid groups (%d groups, %d output channels)", d->groups, d->co); return PCB_ERR_INVALID_ARGUMENT; }
    if (d->groups != 1 && (d->data_format != PCB_LAYOUT_NCHW || d->filter_layout != PCB_FILTER_OIHW)) {
        set_error("grouped convolution takes NCHW tensors and OIHW filters only (groups = %d)", d->groups);
        return PCB_ERR_UNSUPPORTED;
    }
    if (d->dilation_h < 1 || d->dilation_w < 1) { set_error("dilation must be >= 1"); return PCB_ERR_INVALID_ARGUMENT; }
    if (d->variant != PCB_VARIANT_16_PRODUCT && d->variant != PCB_VARIANT_8_PRODUCT) { set_error("unknown variant"); return PCB_ERR_INVALID_ARGUMENT; }
    if (!algebra_setup(d->algebra, g)) { set_error("unknown algebra %d", d->algebra); return PCB_ERR_INVALID_ARGUMENT; }
    // groups: the descriptor's ci is the filters' input channels (the input tensor holds ci * groups), co the total
    g.groups = d->groups;
    g.Nb = d->n; g.Ci = d->ci; g.Co = d->co / d->groups; g.H = d->h; g.W = d->w;
    g.KH = d->kh; g.KW = d->kw; g.SH = d->stride_h; g.SW = d->stride_w; g.DH = d->dilation_h; g.DW = d->dilation_w;
    g.PT = d->pad_top; g.PL = d->pad_left;
    g.HO = out_size(d->h, d->kh, d->dilation_h, d->stride_h, d->pad_top, d->pad_bottom);
    g.WO = out_size(d->w, d->kw, d->dilation_w, d->stride_w, d->pad_left, d->pad_right);
    if (g.HO <= 0 || g.WO <= 0) { set_error("empty convolution output (%d x %d)", g.HO, g.WO); return PCB_ERR_INVALID_ARGUMENT; }
    g.w_io = 0; g.dw_io = 0; g.real_in = d->real_valued_input ? 1 : 0; g.has_bias = d->has_bias ? 1 : 0;
    if (d->data_format < PCB_LAYOUT_NCHW || d->data_format > PCB_LAYOUT_NHWC || d->filter_layout < PCB_FILTER_OIHW || d->filter_layout > PCB_FILTER_HWIO) {
        set_error("unknown tensor layout (data format %d, filter layout %d)", d->data_format, d->filter_layout);
        return PCB_ERR_INVALID_ARGUMENT;
    }
    set_conv_strides(g, d->data_format, d->filter_layout, g.Ci * g.groups, g.Co * g.groups);
    g.plain = (d->data_format == PCB_LAYOUT_NCHW && d->filter_layout == PCB_FILTER_OIHW && g.groups == 1) ? 1 : 0;
    const long long xn = (long long)(g.real_in ? 1 : g.nc) * g.Nb * g.Ci * g.groups * g.H * g.W;
    const long long yn = (long long)g.nc * g.Nb * g.Co * g.groups * g.HO * g.WO;
    const long long wn = (long long)g.nc * g.Co * g.groups * g.Ci * g.KH * g.KW;
    if (xn > MAX_NUMEL || yn > MAX_NUMEL || wn > MAX_NUMEL || g.H > 32767 || g.W > 32767) {
        set_error("tensor too large for 32-bit element offsets");
        return PCB_ERR_TOO_LARGE;
    }
    return PCB_OK;
}

int dense_geom(const pcb_dense_desc* d, Geom& g) {
    if (!d) { set_error("null descriptor"); return PCB_ERR_INVALID_ARGUMENT; }
    if (d->dtype < PCB_F32 || d->dtype > PCB_BF16) { set_error("unknown dtype %d", d->dtype); return PCB_ERR_INVALID_ARGUMENT; }
    if (d->batch < 0 || d->in_features <= 0 || d->out_features <= 0) { set_error("invalid dense geometry"); return PCB_ERR_INVALID_ARGUMENT; }
    if (d->variant != PCB_VARIANT_16_PRODUCT && d->variant != PCB_VARIANT_8_PRODUCT) { set_error("unknown variant"); return PCB_ERR_INVALID_ARGUMENT; }
    if (!algebra_setup(d->algebra, g)) { set_error("unknown algebra %d", d->algebra); return PCB_ERR_INVALID_ARGUMENT; }
    g.Nb = d->batch; g.Ci = d->in_features; g.Co = d->out_features;
    g.H = g.W = g.HO = g.WO = 1; g.KH = g.KW = 1; g.SH = g.SW = 1; g.DH = g.DW = 1; g.PT = g.PL = 0;
    g.w_io = d->filter_oi ? 0 : 1;
    g.dw_io = 1;   // both reference backends emit the filter gradient input-major (src/backend/cudnn/dense.hpp:187-195)
    g.real_in = 0; g.has_bias = d->has_bias ? 1 : 0;
    // x [D*B, I], y [D*B, O]; filters [D, I, O] or [D, O, I]; the filter gradient always [D, I, O]
    g.xp = g.Ci; g.xc = 1; g.xh = g.xw = 0; g.yp = g.Co; g.yc = 1; g.yh = g.yw = 0;
    g.wr = g.Ci * g.Co; g.wh = g.ww = 0; g.wo = g.w_io ? 1 : g.Ci; g.wi = g.w_io ? g.Co : 1;
    g.dr = g.wr; g.dkh = g.dkw = 0; g.dco = 1; g.dci = g.Co;
    g.bias_ld = g.Co; g.plain = 1; g.groups = 1;
    if ((long long)g.nc * g.Nb * g.Ci > MAX_NUMEL || (long long)g.nc * g.Nb * g.Co > MAX_NUMEL || (long long)g.nc * g.Ci * g.Co > MAX_NUMEL) {
        set_error("tensor too large for 32-bit element offsets");
        return PCB_ERR_TOO_LARGE;
    }
    return PCB_OK;
}

// The factorised 8-product form exists for quaternions only (reference: src/conv2d.hpp:167, :433); every other
// algebra runs the generic product whatever the variant says.
int variant_for(const Geom& g, int variant) { return g.nc == 4 ? variant : (int)PCB_VARIANT_16_PRODUCT; }

// The formulation the tensor-core kernels are asked for. With PCB_ENGINE_AUTO the 8-product request is read the way the
// reference means it -- "prefer speed to memory" (Context::preferSpeedToMemory, src/backend/backend.hpp:58): where a
// tensor-core kernel exists it is the fast choice (its one formulation needs no lane temporaries either), and the factorised
// kernels keep the problems the tensor cores do not take. PCB_ENGINE_TENSOR and PCB_ENGINE_SIMT take the variant literally.
int tensor_variant(int variant, int engine) { return engine == PCB_ENGINE_AUTO ? (int)PCB_VARIANT_16_PRODUCT : variant; }

// Layout of the caller's workspace: [0, 256) status block (first word: device wait status), then scratch.
constexpr size_t WS_HEADER = 256;

// Clears the device wait status at the start of an API call. Every kernel launched by the call only ORs into the
// word, so pcb_check_device_status afterwards reports an expiry in ANY launch of the call, not just the last one.
int reset_status(void* workspace, size_t ws_bytes, cudaStream_t stream) {
    if (workspace && ws_bytes >= sizeof(int)) PCB_CUDA_TRY(cudaMemsetAsync(workspace, 0, sizeof(int), stream));
    return PCB_OK;
}

// Staged inputs kept by forward calls, by workspace address (host-side bookkeeping; the data itself lives in that workspace).
// A forward call that stages x in the layout its filter gradient reads records (x, problem signature) under its workspace;
// every later call that is given the same workspace erases the record before it writes there. pcb_qconv2d_bwd_kept reads the
// staged copy only when the record still matches its own x and problem, and stages x itself otherwise.
struct KeptInput { const void* x; unsigned long long signature; };
std::mutex g_kept_mutex;
std::unordered_map<const void*, KeptInput> g_kept;

unsigned long long problem_signature(int dtype, const Geom& g) {
    const int v[] = {dtype, g.nc, g.ga, g.real_in, g.Nb, g.Ci, g.Co, g.H, g.W, g.KH, g.KW, g.SH, g.SW, g.DH, g.DW, g.PT, g.PL, g.HO, g.WO};
    unsigned long long h = 1469598103934665603ull;                   // FNV-1a over the geometry
    for (int x : v) { h ^= (unsigned long long)(unsigned)x; h *= 1099511628211ull; }
    return h;
}
void forget_kept(const void* workspace) {
    if (!workspace) return;
    std::lock_guard<std::mutex> lock(g_kept_mutex);
    g_kept.erase(workspace);
}
void remember_kept(const void* workspace, const void* x, unsigned long long signature) {
    std::lock_guard<std::mutex> lock(g_kept_mutex);
    if (g_kept.size() >= 4096) g_kept.clear();                       // bounded: callers that never run the backward pass
    g_kept[workspace] = KeptInput{x, signature};
}
bool kept_matches(const void* workspace, const void* x, unsigned long long signature) {
    std::lock_guard<std::mutex> lock(g_kept_mutex);
    const auto it = g_kept.find(workspace);
    return it != g_kept.end() && it->second.x == x && it->second.signature == signature;
}

size_t workspace_bytes(Pass pass, int dtype, int variant, int engine, const Geom& g) {
    size_t s = simt_scratch_bytes(pass, dtype, variant, g);
    const size_t t = tensor_scratch_bytes(pass, dtype, tensor_variant(variant, engine), engine, g);
    if (t > s) s = t;
    return WS_HEADER + ((s + 255) / 256) * 256;
}

int run_pass(Pass pass, int dtype, int variant, int engine, const Geom& g, const void* a, const void* b, const void* bias,
             void* out, void* workspace, size_t ws_bytes, cudaStream_t stream, const PassExtras* extras = nullptr) {
    forget_kept(workspace);
    const size_t offset = extras ? extras->scratch_offset : 0;       // scratch another pass of the same call still needs
    const size_t need = workspace_bytes(pass, dtype, variant, engine, g) + offset;
    const int tv = tensor_variant(variant, engine);
    const bool needs_ws = need > WS_HEADER || tensor_path_supported(pass, dtype, tv, g);
    if (needs_ws && (workspace == nullptr || ws_bytes < need)) {
        set_error("workspace of %zu bytes required, %zu given", need, workspace ? ws_bytes : (size_t)0);
        return PCB_ERR_WORKSPACE;
    }
    float* scratch = workspace ? reinterpret_cast<float*>(static_cast<char*>(workspace) + WS_HEADER + offset) : nullptr;
    int* status = static_cast<int*>(workspace);
    // the tensor-core kernels move 16-byte chunks of NCHW / OIHW tensors: every tensor (and the workspace) must be 16-byte
    // aligned. Tensors of other layouts and the channel slices of grouped layers are addressed element by element (staged
    // operands, strided stores), so there only the workspace has to be.
    const uintptr_t tensors = g.plain ? (reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out)) : 0;
    const bool aligned = ((tensors | reinterpret_cast<uintptr_t>(workspace)) & 15u) == 0;
    if (engine != PCB_ENGINE_SIMT && aligned && tensor_path_supported(pass, dtype, tv, g)) {
        const int rc = tensor_launch(pass, dtype, tv, g, a, b, bias, out, scratch, status, stream, extras);
        if (rc == PCB_OK && pass == PASS_FWD && forward_keeps_staged_input(dtype, tv, g)) remember_kept(workspace, b, problem_signature(dtype, g));
        return rc;
    }
    if (engine == PCB_ENGINE_TENSOR) {
        set_error("no tensor-core kernel for this problem");
        return PCB_ERR_UNSUPPORTED;
    }
    return simt_launch(pass, dtype, variant, g, a, b, bias, out, scratch, stream);
}

// Grouped convolution (reference: the groups argument of the scalar convolutions, src/backend/cudnn/conv2d.hpp:126-127):
// one pass per group on the CUDA-core kernels, which address every tensor through strides -- a group is a channel slice
// of x, y and the filters. The filter gradient of a group is produced contiguously in the workspace and copied into its
// slice (component r of the gradient is Co_total * Ci * taps elements apart, a group's slice Co * Ci * taps wide).
size_t group_slice_bytes(int dtype, const Geom& g) {
    return (((size_t)g.nc * g.Co * g.Ci * g.KH * g.KW * dtype_size(dtype)) + 255) / 256 * 256;
}

size_t conv_workspace_bytes(Pass pass, int dtype, int variant, int engine, const Geom& g) {
    if (g.groups == 1) return workspace_bytes(pass, dtype, variant, engine, g);
    return workspace_bytes(pass, dtype, variant, engine, g) + (pass == PASS_BWD_FILTER ? group_slice_bytes(dtype, g) : 0);
}

int run_conv_pass(Pass pass, int dtype, int variant, int engine, const Geom& g, const void* a, const void* b, const void* bias,
                  void* out, void* workspace, size_t ws_bytes, cudaStream_t stream, const PassExtras* extras = nullptr) {
    if (g.groups == 1) return run_pass(pass, dtype, variant, engine, g, a, b, bias, out, workspace, ws_bytes, stream, extras);
    const size_t es = dtype_size(dtype);
    const size_t need = conv_workspace_bytes(pass, dtype, variant, engine, g);
    if (need > WS_HEADER && (workspace == nullptr || ws_bytes < need)) {
        set_error("workspace of %zu bytes required, %zu given", need, workspace ? ws_bytes : (size_t)0);
        return PCB_ERR_WORKSPACE;
    }
    const size_t taps = (size_t)g.KH * g.KW;
    const size_t x_step = (size_t)g.Ci * g.H * g.W * es, y_step = (size_t)g.Co * g.HO * g.WO * es;
    const size_t w_step = (size_t)g.Co * g.Ci * taps * es, bias_step = (size_t)g.Co * es;
    const char* ca = static_cast<const char*>(a);
    const char* cb = static_cast<const char*>(b);
    char* co = static_cast<char*>(out);
    for (int gi = 0; gi < g.groups; ++gi) {
        int rc;
        if (pass == PASS_FWD) {            // a = filters, b = x, out = y
            rc = run_pass(pass, dtype, variant, engine, g, ca + gi * w_step, cb + gi * x_step,
                          bias ? static_cast<const char*>(bias) + gi * bias_step : nullptr, co + gi * y_step, workspace, ws_bytes, stream);
        } else if (pass == PASS_BWD_DATA) { // a = filters, b = dy, out = dx
            rc = run_pass(pass, dtype, variant, engine, g, ca + gi * w_step, cb + gi * y_step, nullptr, co + gi * x_step, workspace, ws_bytes, stream);
        } else {                           // a = dy, b = x, out = dw: contiguous slice first
            Geom gs = g;
            gs.dr = g.Co * g.Ci * (int)taps;
            const size_t inner = workspace_bytes(pass, dtype, variant, engine, g);   // a multiple of 256 bytes
            char* tmp = static_cast<char*>(workspace) + inner;                             // the slice follows the pass's own scratch
            rc = run_pass(pass, dtype, variant, engine, gs, ca + gi * y_step, cb + gi * x_step, nullptr, tmp, workspace, inner, stream);
            if (rc == PCB_OK) {
                const size_t row = (size_t)g.Co * g.Ci * taps * es;
                PCB_CUDA_TRY(cudaMemcpy2DAsync(co + gi * w_step, row * g.groups, tmp, row, row, g.nc, cudaMemcpyDeviceToDevice, stream));
            }
        }
        if (rc != PCB_OK) return rc;
    }
    return PCB_OK;
}

// One thread waits, with the given clock limit, on an mbarrier that nothing ever signals: the wait runs out, the
// status word gets its bit and the kernel returns normally. No tensor memory, no copies, nothing left in flight.
constexpr int ST_SELFTEST = 0x40000000;
__global__ void wait_expiry_kernel(int* status, long long limit_clocks) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        umma::mbar_init(umma::smem_u32(&bar), 1);
        umma::fence_barrier_init();
        umma::mbar_wait_bounded(umma::smem_u32(&bar), 0, status, ST_SELFTEST, limit_clocks);
    }
}

// The three convolution passes without the status reset (an API call clears the word once, then runs one or more of these).
int conv_fwd(const pcb_conv2d_desc* desc, const void* x, const void* w, const void* bias, void* y,
             void* workspace, size_t workspace_bytes_, cudaStream_t stream) {
    Geom g;
    int rc = conv_geom(desc, g);
    if (rc != PCB_OK) return rc;
    if (g.Nb == 0) return PCB_OK;   // empty input: silent no-op, as the reference (src/conv2d.hpp:81-82)
    if (!x || !w || !y || (g.has_bias && !bias)) { set_error("null tensor pointer"); return PCB_ERR_INVALID_ARGUMENT; }
    if (g.real_in && g.has_bias) { set_error("bias addition is not supported for real-valued inputs"); return PCB_ERR_UNSUPPORTED; }
    return run_conv_pass(PASS_FWD, desc->dtype, variant_for(g, desc->variant), desc->engine, g, w, x, bias, y, workspace, workspace_bytes_, stream);
}

int conv_bwd_data(const pcb_conv2d_desc* desc, const void* w, const void* dy, void* dx,
                  void* workspace, size_t workspace_bytes_, cudaStream_t stream) {
    Geom g;
    int rc = conv_geom(desc, g);
    if (rc != PCB_OK) return rc;
    if (g.Nb == 0) return PCB_OK;
    if (g.real_in) { set_error("input gradient required for a real-valued input tensor"); return PCB_ERR_UNSUPPORTED; }
    if (!w || !dy || !dx) { set_error("null tensor pointer"); return PCB_ERR_INVALID_ARGUMENT; }
    return run_conv_pass(PASS_BWD_DATA, desc->dtype, variant_for(g, desc->variant), desc->engine, g, w, dy, nullptr, dx, workspace, workspace_bytes_, stream);
}

int conv_bwd_filter(const pcb_conv2d_desc* desc, const void* x, const void* dy, void* dw,
                    void* workspace, size_t workspace_bytes_, cudaStream_t stream, const PassExtras* extras = nullptr) {
    Geom g;
    int rc = conv_geom(desc, g);
    if (rc != PCB_OK) return rc;
    if (!dw) { set_error("null tensor pointer"); return PCB_ERR_INVALID_ARGUMENT; }
    if (g.Nb == 0) {   // empty input: zero filter gradient, as the reference (src/conv2d.hpp:341-344)
        PCB_CUDA_TRY(cudaMemsetAsync(dw, 0, (size_t)g.nc * g.Co * g.groups * g.Ci * g.KH * g.KW * dtype_size(desc->dtype), stream));
        return PCB_OK;
    }
    if (!x || !dy) { set_error("null tensor pointer"); return PCB_ERR_INVALID_ARGUMENT; }
    return run_conv_pass(PASS_BWD_FILTER, desc->dtype, variant_for(g, desc->variant), desc->engine, g, dy, x, nullptr, dw, workspace, workspace_bytes_, stream, extras);
}

// Staged dy shared by the two gradients of one call: the padded copy that backward-data makes at the start of the scratch
// stays where it is, and the filter gradient -- run second, its own scratch placed behind that copy -- reads it through a
// tensor map instead of staging dy again. Applies to 16-bit stride-1 tapped layers whose two kernels agree on the layout.
bool bwd_shares_dy(const pcb_conv2d_desc* desc, const Geom& g, StagedView* view, size_t* offset) {
    if (desc->engine == PCB_ENGINE_SIMT || !desc->require_input_grad || g.Nb == 0 || g.groups != 1) return false;
    size_t bytes = 0;
    if (!backward_shares_staged_dy(desc->dtype, tensor_variant(variant_for(g, desc->variant), desc->engine), g, view, &bytes)) return false;
    *offset = (bytes + 1023) / 1024 * 1024;
    return true;
}

// dw and dx of one call. `kept_x`: see pcb_qconv2d_bwd_kept.
int conv_bwd_both(const pcb_conv2d_desc* desc, const void* x, const void* w, const void* dy, void* dw, void* dx,
                  void* workspace, size_t workspace_bytes_, cudaStream_t stream, const void* kept_x) {
    Geom g;
    int rc = conv_geom(desc, g);
    if (rc != PCB_OK) return rc;
    PassExtras extras;
    extras.kept_x = kept_x;
    StagedView view;
    size_t offset = 0;
    const uintptr_t all = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(dy) |
                          reinterpret_cast<uintptr_t>(dw) | reinterpret_cast<uintptr_t>(dx) | reinterpret_cast<uintptr_t>(workspace);
    if (x && w && dy && dw && dx && workspace && (all & 15u) == 0 && bwd_shares_dy(desc, g, &view, &offset) &&
        workspace_bytes_ >= conv_workspace_bytes(PASS_BWD_FILTER, desc->dtype, variant_for(g, desc->variant), desc->engine, g) + offset) {
        // backward-data first: it leaves the padded dy in [WS_HEADER, WS_HEADER + offset)
        rc = conv_bwd_data(desc, w, dy, dx, workspace, workspace_bytes_, stream);
        if (rc != PCB_OK) return rc;
        view.base = static_cast<const char*>(workspace) + WS_HEADER;
        extras.dy = view;
        extras.scratch_offset = offset;
        return conv_bwd_filter(desc, x, dy, dw, workspace, workspace_bytes_, stream, &extras);
    }
    rc = conv_bwd_filter(desc, x, dy, dw, workspace, workspace_bytes_, stream, &extras);
    if (rc != PCB_OK) return rc;
    if (desc->require_input_grad && desc->n > 0) rc = conv_bwd_data(desc, w, dy, dx, workspace, workspace_bytes_, stream);
    return rc;
}

}  // namespace
}  // namespace pcb

using namespace pcb;

extern "C" {

int pcb_set_sm_margin(int sms) {
    if (sms < 0 || sms > 64) return PCB_ERR_INVALID_ARGUMENT;
    pcb::g_sm_margin = sms;
    return PCB_OK;
}
int pcb_get_sm_margin(void) { return pcb::g_sm_margin; }


const char* pcb_version(void) { return "phoenix_core_b200 0.1 (sm_100a)"; }

const char* pcb_status_string(int status) {
    switch (status) {
        case PCB_OK: return "ok";
        case PCB_ERR_INVALID_ARGUMENT: return "invalid argument";
        case PCB_ERR_UNSUPPORTED: return "unsupported configuration";
        case PCB_ERR_WORKSPACE: return "workspace missing or too small";
        case PCB_ERR_CUDA: return "CUDA runtime error";
        case PCB_ERR_DEVICE_TIMEOUT: return "device-side wait expired";
        case PCB_ERR_TOO_LARGE: return "size beyond supported maximum";
    }
    return "unknown status";
}

const char* pcb_last_error_message(void) { return g_error; }

int pcb_conv2d_output_size(const pcb_conv2d_desc* desc, int32_t* out_h, int32_t* out_w) {
    Geom g;
    const int rc = conv_geom(desc, g);
    if (rc != PCB_OK) return rc;
    if (out_h) *out_h = g.HO;
    if (out_w) *out_w = g.WO;
    return PCB_OK;
}

size_t pcb_qconv2d_fwd_workspace_size(const pcb_conv2d_desc* desc) {
    Geom g;
    if (conv_geom(desc, g) != PCB_OK) return 0;
    return conv_workspace_bytes(PASS_FWD, desc->dtype, variant_for(g, desc->variant), desc->engine, g);
}

size_t pcb_qconv2d_bwd_workspace_size(const pcb_conv2d_desc* desc) {
    Geom g;
    if (conv_geom(desc, g) != PCB_OK) return 0;
    const size_t a = conv_workspace_bytes(PASS_BWD_DATA, desc->dtype, variant_for(g, desc->variant), desc->engine, g);
    size_t b = conv_workspace_bytes(PASS_BWD_FILTER, desc->dtype, variant_for(g, desc->variant), desc->engine, g);
    StagedView view;
    size_t offset = 0;
    if (bwd_shares_dy(desc, g, &view, &offset)) b += offset;          // the filter gradient's scratch lies behind the shared copy of dy
    return a > b ? a : b;
}

size_t pcb_qdense_fwd_workspace_size(const pcb_dense_desc* desc) {
    Geom g;
    if (dense_geom(desc, g) != PCB_OK) return 0;
    return workspace_bytes(PASS_FWD, desc->dtype, variant_for(g, desc->variant), desc->engine, g);
}

size_t pcb_qdense_bwd_workspace_size(const pcb_dense_desc* desc) {
    Geom g;
    if (dense_geom(desc, g) != PCB_OK) return 0;
    const size_t a = workspace_bytes(PASS_BWD_DATA, desc->dtype, variant_for(g, desc->variant), desc->engine, g);
    const size_t b = workspace_bytes(PASS_BWD_FILTER, desc->dtype, variant_for(g, desc->variant), desc->engine, g);
    return a > b ? a : b;
}

int pcb_qconv2d_fwd(const pcb_conv2d_desc* desc, const void* x, const void* w, const void* bias, void* y,
                    void* workspace, size_t workspace_bytes_, void* stream) {
    const int rc = reset_status(workspace, workspace_bytes_, (cudaStream_t)stream);
    return rc != PCB_OK ? rc : conv_fwd(desc, x, w, bias, y, workspace, workspace_bytes_, (cudaStream_t)stream);
}

int pcb_qconv2d_bwd_data(const pcb_conv2d_desc* desc, const void* w, const void* dy, void* dx,
                         void* workspace, size_t workspace_bytes_, void* stream) {
    const int rc = reset_status(workspace, workspace_bytes_, (cudaStream_t)stream);
    return rc != PCB_OK ? rc : conv_bwd_data(desc, w, dy, dx, workspace, workspace_bytes_, (cudaStream_t)stream);
}

int pcb_qconv2d_bwd_filter(const pcb_conv2d_desc* desc, const void* x, const void* dy, void* dw,
                           void* workspace, size_t workspace_bytes_, void* stream) {
    const int rc = reset_status(workspace, workspace_bytes_, (cudaStream_t)stream);
    return rc != PCB_OK ? rc : conv_bwd_filter(desc, x, dy, dw, workspace, workspace_bytes_, (cudaStream_t)stream);
}

int pcb_qconv2d_bwd_filter_noalloc(const pcb_conv2d_desc* desc, const void* x, const void* dy, void* dw, void* stream) {
    Geom g;
    int rc = conv_geom(desc, g);
    if (rc != PCB_OK) return rc;
    if (!dw) { set_error("null tensor pointer"); return PCB_ERR_INVALID_ARGUMENT; }
    if (g.groups != 1) { set_error("the allocation-free filter gradient takes one group"); return PCB_ERR_UNSUPPORTED; }
    if ((size_t)g.nc * g.Co * g.Ci * g.KH * g.KW > simt_static_scratch_capacity()) {
        set_error("filter gradient of %zu elements exceeds the built-in scratch of %zu elements",
                  (size_t)g.nc * g.Co * g.Ci * g.KH * g.KW, simt_static_scratch_capacity());
        return PCB_ERR_TOO_LARGE;
    }
    if (g.Nb == 0) {
        PCB_CUDA_TRY(cudaMemsetAsync(dw, 0, (size_t)g.nc * g.Co * g.Ci * g.KH * g.KW * dtype_size(desc->dtype), (cudaStream_t)stream));
        return PCB_OK;
    }
    if (!x || !dy) { set_error("null tensor pointer"); return PCB_ERR_INVALID_ARGUMENT; }
    return simt_bwd_filter_static(desc->dtype, variant_for(g, desc->variant), g, dy, x, dw, (cudaStream_t)stream);
}

int pcb_qconv2d_bwd(const pcb_conv2d_desc* desc, const void* x, const void* w, const void* dy, void* dw, void* dx,
                    void* workspace, size_t workspace_bytes_, void* stream) {
    const int rc = reset_status(workspace, workspace_bytes_, (cudaStream_t)stream);
    if (rc != PCB_OK) return rc;
    return conv_bwd_both(desc, x, w, dy, dw, dx, workspace, workspace_bytes_, (cudaStream_t)stream, nullptr);
}

int pcb_qconv2d_fwd_keeps_input(const pcb_conv2d_desc* desc) {
    Geom g;
    if (conv_geom(desc, g) != PCB_OK || desc->engine == PCB_ENGINE_SIMT || g.Nb == 0) return 0;
    return forward_keeps_staged_input(desc->dtype, tensor_variant(variant_for(g, desc->variant), desc->engine), g) ? 1 : 0;
}

int pcb_qconv2d_bwd_kept(const pcb_conv2d_desc* desc, const void* x, const void* w, const void* dy, void* dw, void* dx,
                         const void* fwd_workspace, size_t fwd_workspace_bytes, void* workspace, size_t workspace_bytes_, void* stream) {
    int rc = reset_status(workspace, workspace_bytes_, (cudaStream_t)stream);
    if (rc != PCB_OK) return rc;
    const void* kept_x = nullptr;
    Geom g;
    if (fwd_workspace && fwd_workspace != workspace && (reinterpret_cast<uintptr_t>(fwd_workspace) & 15u) == 0 && conv_geom(desc, g) == PCB_OK &&
        pcb_qconv2d_fwd_keeps_input(desc) && fwd_workspace_bytes >= pcb_qconv2d_fwd_workspace_size(desc) &&
        kept_matches(fwd_workspace, x, problem_signature(desc->dtype, g)))
        kept_x = static_cast<const char*>(fwd_workspace) + WS_HEADER;
    return conv_bwd_both(desc, x, w, dy, dw, dx, workspace, workspace_bytes_, (cudaStream_t)stream, kept_x);
}

int pcb_qdense_fwd(const pcb_dense_desc* desc, const void* x, const void* w, const void* bias, void* y,
                   void* workspace, size_t workspace_bytes_, void* stream) {
    Geom g;
    int rc = dense_geom(desc, g);
    if (rc != PCB_OK) return rc;
    if (g.Nb == 0) return PCB_OK;
    if (!x || !w || !y || (g.has_bias && !bias)) { set_error("null tensor pointer"); return PCB_ERR_INVALID_ARGUMENT; }
    rc = reset_status(workspace, workspace_bytes_, (cudaStream_t)stream);
    if (rc != PCB_OK) return rc;
    return run_pass(PASS_FWD, desc->dtype, variant_for(g, desc->variant), desc->engine, g, w, x, bias, y, workspace, workspace_bytes_, (cudaStream_t)stream);
}

int pcb_qdense_bwd(const pcb_dense_desc* desc, const void* x, const void* w, const void* dy, void* dw, void* dx,
                   void* workspace, size_t workspace_bytes_, void* stream) {
    Geom g;
    int rc = dense_geom(desc, g);
    if (rc != PCB_OK) return rc;
    if (!dw) { set_error("null tensor pointer"); return PCB_ERR_INVALID_ARGUMENT; }
    if (g.Nb == 0) {   // src/dense.hpp:226-229
        PCB_CUDA_TRY(cudaMemsetAsync(dw, 0, (size_t)g.nc * g.Co * g.Ci * dtype_size(desc->dtype), (cudaStream_t)stream));
        return PCB_OK;
    }
    if (!x || !w || !dy || (desc->require_input_grad && !dx)) { set_error("null tensor pointer"); return PCB_ERR_INVALID_ARGUMENT; }
    rc = reset_status(workspace, workspace_bytes_, (cudaStream_t)stream);
    if (rc != PCB_OK) return rc;
    rc = run_pass(PASS_BWD_FILTER, desc->dtype, variant_for(g, desc->variant), desc->engine, g, dy, x, nullptr, dw, workspace, workspace_bytes_, (cudaStream_t)stream);
    if (rc != PCB_OK) return rc;
    if (desc->require_input_grad)
        rc = run_pass(PASS_BWD_DATA, desc->dtype, variant_for(g, desc->variant), desc->engine, g, w, dy, nullptr, dx, workspace, workspace_bytes_, (cudaStream_t)stream);
    return rc;
}

int pcb_qconv2d_engine_for(const pcb_conv2d_desc* desc, int pass) {
    Geom g;
    const int rc = conv_geom(desc, g);
    if (rc != PCB_OK) return rc;
    if (pass < 0 || pass > 2) { set_error("pass must be 0, 1 or 2"); return PCB_ERR_INVALID_ARGUMENT; }
    if (desc->engine != PCB_ENGINE_SIMT && tensor_path_supported((Pass)pass, desc->dtype, tensor_variant(variant_for(g, desc->variant), desc->engine), g)) return PCB_ENGINE_TENSOR;
    return desc->engine == PCB_ENGINE_TENSOR ? (int)PCB_ERR_UNSUPPORTED : (int)PCB_ENGINE_SIMT;
}

int pcb_qdense_engine_for(const pcb_dense_desc* desc, int pass) {
    Geom g;
    const int rc = dense_geom(desc, g);
    if (rc != PCB_OK) return rc;
    if (pass < 0 || pass > 2) { set_error("pass must be 0, 1 or 2"); return PCB_ERR_INVALID_ARGUMENT; }
    if (desc->engine != PCB_ENGINE_SIMT && tensor_path_supported((Pass)pass, desc->dtype, tensor_variant(variant_for(g, desc->variant), desc->engine), g)) return PCB_ENGINE_TENSOR;
    return desc->engine == PCB_ENGINE_TENSOR ? (int)PCB_ERR_UNSUPPORTED : (int)PCB_ENGINE_SIMT;
}

int pcb_selftest_wait_expiry(const pcb_conv2d_desc* desc, const void* x, const void* w, void* y, void* workspace,
                             size_t workspace_bytes_, long long limit_clocks, void* stream) {
    if (!workspace || workspace_bytes_ < WS_HEADER) { set_error("the self-test needs a workspace"); return PCB_ERR_WORKSPACE; }
    if (limit_clocks < 1 || limit_clocks > (1ll << 24)) { set_error("limit_clocks must be in [1, 2^24]"); return PCB_ERR_INVALID_ARGUMENT; }
    int rc = reset_status(workspace, workspace_bytes_, (cudaStream_t)stream);
    if (rc != PCB_OK) return rc;
    wait_expiry_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(static_cast<int*>(workspace), limit_clocks);
    PCB_CUDA_TRY(cudaGetLastError());
    // a further launch of the same call: it must leave the recorded expiry in place
    if (desc) rc = conv_fwd(desc, x, w, nullptr, y, workspace, workspace_bytes_, (cudaStream_t)stream);
    return rc;
}

int pcb_check_device_status(const void* workspace, size_t workspace_bytes_, void* stream) {
    if (!workspace || workspace_bytes_ < sizeof(int)) return PCB_OK;
    int word = 0;
    PCB_CUDA_TRY(cudaMemcpyAsync(&word, workspace, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    PCB_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
    if (word != 0) {
        set_error("device-side wait expired (status word 0x%08x)", word);
        return PCB_ERR_DEVICE_TIMEOUT;
    }
    return PCB_OK;
}

}  // extern "C"

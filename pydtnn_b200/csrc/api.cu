// C ABI of the convolution / FC path: argument checking, engine selection, dispatch.
#include "b2c_common.cuh"
#include <string.h>

namespace b2c {
static thread_local char g_cuda_err[256] = "";
static unsigned long long g_launches = 0;
void count_launch() { __atomic_add_fetch(&g_launches, 1ULL, __ATOMIC_RELAXED); }
void set_cuda_error(cudaError_t e, const char* where) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s", where, cudaGetErrorString(e));
}

// Shapes the tensor-core kernels accept but the FMA engine runs faster (measured on fully connected layers at
// batch 32-64): a weight gradient summed over a handful of pixels is an outer product bound by writing dw, which the
// FMA engine's dense kernel does at HBM speed; a GEMM with one 128-row tile and at most eight column tiles leaves
// each tile to ~18 CTAs of the balanced mode, whose partial tiles the owner adds one after the other.
static bool fma_is_faster(const Geo& g, int pass) {
    const bool one_pixel_images = g.h == 1 && g.w == 1 && g.kh == 1 && g.kw == 1 && g.vpad == 0 && g.hpad == 0;
    if (!one_pixel_images || g.n > 128) return false;
    if (pass == B2C_PASS_WGRAD) return true;
    return (pass == B2C_PASS_FPROP ? g.co : g.ci) <= 1024;
}

// FMA for everything unless the tensor-core engine takes the shape (AUTO) or is forced.
static int pick_engine(const Geo& g, int pass, int& engine) {
    bool tc = tc_supported(g, pass);
    if (g.engine == B2C_ENGINE_AUTO && tc && fma_is_faster(g, pass)) tc = false;
    if (g.engine == B2C_ENGINE_TENSOR) { if (!tc) return B2C_ERR_UNSUPPORTED; engine = B2C_ENGINE_TENSOR; }
    else if (g.engine == B2C_ENGINE_FMA) engine = B2C_ENGINE_FMA;
    else engine = tc ? B2C_ENGINE_TENSOR : B2C_ENGINE_FMA;
    return B2C_OK;
}

// An FC layer is a 1x1 convolution over a (batch, 1, 1, in) NHWC tensor with a (in,1,1,out) filter.
static int fc_geo(int dtype, int engine, int batch, int in_f, int out_f, Geo& g) {
    b2c_conv_desc d{};
    d.layout = B2C_LAYOUT_NHWC; d.dtype = dtype; d.w_layout = B2C_W_CRSK; d.engine = engine;
    d.n = batch; d.h = 1; d.w = 1; d.ci = in_f; d.co = out_f; d.kh = 1; d.kw = 1;
    d.vstr = d.hstr = d.vdil = d.hdil = 1;
    return make_geo(&d, g);
}
}  // namespace b2c

using namespace b2c;

extern "C" const char* b2c_status_string(int status) {
    switch (status) {
        case B2C_OK: return "ok";
        case B2C_ERR_NULL_POINTER: return "null pointer argument";
        case B2C_ERR_BAD_GEOMETRY: return "invalid geometry (non-positive size, empty output, or stride/dilation < 1)";
        case B2C_ERR_BAD_ENUM: return "layout / dtype / weight layout / engine / pass out of range";
        case B2C_ERR_WORKSPACE_TOO_SMALL: return "workspace too small or missing";
        case B2C_ERR_MISALIGNED: return "pointer not aligned as required";
        case B2C_ERR_UNSUPPORTED: return "shape not supported by the requested engine";
        case B2C_ERR_CUDA: return "CUDA launch error";
        case B2C_ERR_TOO_LARGE: return "size exceeds a fixed capacity";
        case B2C_ERR_DEVICE_TIMEOUT: return "a bounded in-kernel wait ran out";
        default: return "unknown status";
    }
}
extern "C" const char* b2c_last_cuda_error(void) { return g_cuda_err; }
extern "C" int b2c_version(void) { return 100; }
extern "C" uint64_t b2c_launch_count(void) { return (uint64_t)__atomic_load_n(&b2c::g_launches, __ATOMIC_RELAXED); }

extern "C" int b2c_check_device_status(int* detail) {
    int v = 0;
    int rc = tc_read_status(&v);
    if (detail) *detail = v;
    if (rc) return rc;
    return v ? B2C_ERR_DEVICE_TIMEOUT : B2C_OK;
}

extern "C" int b2c_selftest_bounded_wait(int64_t limit_cycles, void* stream) {
    return tc_wait_selftest((long long)limit_cycles, (cudaStream_t)stream);
}

extern "C" int b2c_conv_engine_for(const b2c_conv_desc* desc, int pass) {
    Geo g; int rc = make_geo(desc, g); if (rc) return rc;
    if (pass < 0 || pass > 2) return B2C_ERR_BAD_ENUM;
    int e; rc = pick_engine(g, pass, e); if (rc) return rc;
    return e;
}

extern "C" size_t b2c_conv_workspace_bytes(const b2c_conv_desc* desc, int pass) {
    Geo g; if (make_geo(desc, g)) return 0;
    if (pass < 0 || pass > 2) return 0;
    int e; if (pick_engine(g, pass, e)) return 0;
    return e == B2C_ENGINE_TENSOR ? tc_workspace_bytes(g, pass) : fma_workspace_bytes(g, pass);
}

extern "C" int b2c_conv_fprop(const b2c_conv_desc* desc, const void* x, const void* w, const void* bias,
                              const b2c_bn_params* bn, int relu, void* y, void* ws, size_t ws_bytes, void* stream) {
    Geo g; int rc = make_geo(desc, g); if (rc) return rc;
    if (!x || !w || !y) return B2C_ERR_NULL_POINTER;
    if (bn && (!bn->mean || !bn->inv_std || !bn->gamma || !bn->beta)) return B2C_ERR_NULL_POINTER;
    int e; rc = pick_engine(g, B2C_PASS_FPROP, e); if (rc) return rc;
    if (e == B2C_ENGINE_TENSOR) return tc_fprop(g, x, w, bias, bn, relu, y, ws, ws_bytes, (cudaStream_t)stream);
    return fma_fprop(g, x, w, bias, bn, relu, y, ws, ws_bytes, (cudaStream_t)stream);
}

extern "C" size_t b2c_conv_stats_bytes(const b2c_conv_desc* desc) {
    Geo g; if (make_geo(desc, g)) return 0;
    if (g.dtype != B2C_F32) return 0;
    int e; if (pick_engine(g, B2C_PASS_FPROP, e) || e != B2C_ENGINE_TENSOR) return 0;
    return tc_stats_bytes(g);
}

extern "C" int b2c_conv_fprop_stats(const b2c_conv_desc* desc, const void* x, const void* w, const void* bias, void* y,
                                    void* stats, size_t stats_bytes, void* ws, size_t ws_bytes, void* stream) {
    Geo g; int rc = make_geo(desc, g); if (rc) return rc;
    if (!x || !w || !y || !stats) return B2C_ERR_NULL_POINTER;
    if (g.dtype != B2C_F32) return B2C_ERR_UNSUPPORTED;
    int e; rc = pick_engine(g, B2C_PASS_FPROP, e); if (rc) return rc;
    if (e != B2C_ENGINE_TENSOR) return B2C_ERR_UNSUPPORTED;
    return tc_fprop_stats(g, x, w, bias, y, stats, stats_bytes, ws, ws_bytes, (cudaStream_t)stream);
}

extern "C" int b2c_conv_dgrad(const b2c_conv_desc* desc, const void* dy, const void* w, void* dx,
                              void* ws, size_t ws_bytes, void* stream) {
    Geo g; int rc = make_geo(desc, g); if (rc) return rc;
    if (!dy || !w || !dx) return B2C_ERR_NULL_POINTER;
    int e; rc = pick_engine(g, B2C_PASS_DGRAD, e); if (rc) return rc;
    if (e == B2C_ENGINE_TENSOR) return tc_dgrad(g, dy, w, dx, ws, ws_bytes, (cudaStream_t)stream);
    return fma_dgrad(g, dy, w, dx, ws, ws_bytes, (cudaStream_t)stream);
}

extern "C" int b2c_conv_keeps_lowered_input(const b2c_conv_desc* desc) {
    Geo g; if (make_geo(desc, g)) return 0;
    int e; if (pick_engine(g, B2C_PASS_WGRAD, e) || e != B2C_ENGINE_TENSOR) return 0;
    if (pick_engine(g, B2C_PASS_FPROP, e) || e != B2C_ENGINE_TENSOR) return 0;
    return tc_keeps_lowered(g) ? 1 : 0;
}

extern "C" int b2c_conv_wgrad_lowered(const b2c_conv_desc* desc, const void* x, const void* dy, void* dw, void* db,
                                      void* ws, size_t ws_bytes, void* stream) {
    Geo g; int rc = make_geo(desc, g); if (rc) return rc;
    if (!x || !dy || !dw) return B2C_ERR_NULL_POINTER;
    int e; rc = pick_engine(g, B2C_PASS_WGRAD, e); if (rc) return rc;
    if (e != B2C_ENGINE_TENSOR) return B2C_ERR_UNSUPPORTED;
    return tc_wgrad_lowered(g, x, dy, dw, db, ws, ws_bytes, (cudaStream_t)stream);
}

extern "C" int b2c_conv_wgrad(const b2c_conv_desc* desc, const void* x, const void* dy, void* dw, void* db,
                              void* ws, size_t ws_bytes, void* stream) {
    Geo g; int rc = make_geo(desc, g); if (rc) return rc;
    if (!x || !dy || !dw) return B2C_ERR_NULL_POINTER;
    int e; rc = pick_engine(g, B2C_PASS_WGRAD, e); if (rc) return rc;
    if (e == B2C_ENGINE_TENSOR) return tc_wgrad(g, x, dy, dw, db, ws, ws_bytes, (cudaStream_t)stream);
    return fma_wgrad(g, x, dy, dw, db, ws, ws_bytes, (cudaStream_t)stream);
}

extern "C" int b2c_conv_index_map(const b2c_conv_desc* desc, int64_t* map, void* stream) {
    Geo g; int rc = make_geo(desc, g); if (rc) return rc;
    if (!map) return B2C_ERR_NULL_POINTER;
    return fma_index_map(g, map, (cudaStream_t)stream);
}

extern "C" size_t b2c_fc_workspace_bytes(int dtype, int batch, int in_f, int out_f, int engine) {
    Geo g; if (fc_geo(dtype, engine, batch, in_f, out_f, g)) return 0;
    size_t m = 0;
    for (int pass = 0; pass < 3; pass++) {
        int e; if (pick_engine(g, pass, e)) return 0;
        size_t b = e == B2C_ENGINE_TENSOR ? tc_workspace_bytes(g, pass) : fma_workspace_bytes(g, pass);
        if (b > m) m = b;
    }
    if (tc_fc_small_batch(dtype, engine, batch, in_f, out_f)) {
        size_t b = tc_fc_small_batch_bytes(batch, in_f, out_f);
        if (b > m) m = b;
    }
    return m;
}

extern "C" int b2c_fc_forward(int dtype, int engine, int batch, int in_f, int out_f, const void* x, const void* w,
                              const void* bias, void* y, void* ws, size_t ws_bytes, void* stream) {
    Geo g; int rc = fc_geo(dtype, engine, batch, in_f, out_f, g); if (rc) return rc;
    if (!x || !w || !y) return B2C_ERR_NULL_POINTER;
    if (tc_fc_small_batch(dtype, engine, batch, in_f, out_f))
        return tc_fc_forward_small_batch(batch, in_f, out_f, x, w, bias, y, ws, ws_bytes, (cudaStream_t)stream);
    int e; rc = pick_engine(g, B2C_PASS_FPROP, e); if (rc) return rc;
    if (e == B2C_ENGINE_TENSOR) return tc_fprop(g, x, w, bias, nullptr, 0, y, ws, ws_bytes, (cudaStream_t)stream);
    return fma_fprop(g, x, w, bias, nullptr, 0, y, ws, ws_bytes, (cudaStream_t)stream);
}

extern "C" int b2c_fc_backward(int dtype, int engine, int batch, int in_f, int out_f, const void* x, const void* dy,
                               const void* w, void* dw, void* db, void* dx, void* ws, size_t ws_bytes, void* stream) {
    Geo g; int rc = fc_geo(dtype, engine, batch, in_f, out_f, g); if (rc) return rc;
    if (!dy) return B2C_ERR_NULL_POINTER;
    cudaStream_t st = (cudaStream_t)stream;
    if (tc_fc_small_batch(dtype, engine, batch, in_f, out_f)) {
        if (dw) {
            if (!x) return B2C_ERR_NULL_POINTER;
            rc = tc_fc_wgrad_small_batch(batch, in_f, out_f, x, dy, dw, db, ws, ws_bytes, st); if (rc) return rc;
        } else if (db) {
            if (!ws || ws_bytes < channel_sum_workspace_bytes(batch, out_f, 1)) return B2C_ERR_WORKSPACE_TOO_SMALL;
            rc = channel_sum(dtype, B2C_LAYOUT_NHWC, batch, out_f, 1, dy, db, ws, ws_bytes, st); if (rc) return rc;
        }
        if (dx) {
            if (!w) return B2C_ERR_NULL_POINTER;
            rc = tc_fc_dgrad_small_batch(batch, in_f, out_f, dy, w, dx, ws, ws_bytes, st);
        }
        return rc;
    }
    if (dw) {
        if (!x) return B2C_ERR_NULL_POINTER;
        int e; rc = pick_engine(g, B2C_PASS_WGRAD, e); if (rc) return rc;
        rc = e == B2C_ENGINE_TENSOR ? tc_wgrad(g, x, dy, dw, db, ws, ws_bytes, st) : fma_wgrad(g, x, dy, dw, db, ws, ws_bytes, st);
        if (rc) return rc;
    } else if (db) {
        size_t need = channel_sum_workspace_bytes(batch, out_f, 1);
        if (!ws || ws_bytes < need) return B2C_ERR_WORKSPACE_TOO_SMALL;
        rc = channel_sum(dtype, B2C_LAYOUT_NHWC, batch, out_f, 1, dy, db, ws, ws_bytes, st); if (rc) return rc;
    }
    if (dx) {
        if (!w) return B2C_ERR_NULL_POINTER;
        int e; rc = pick_engine(g, B2C_PASS_DGRAD, e); if (rc) return rc;
        rc = e == B2C_ENGINE_TENSOR ? tc_dgrad(g, dy, w, dx, ws, ws_bytes, st) : fma_dgrad(g, dy, w, dx, ws, ws_bytes, st);
    }
    return rc;
}

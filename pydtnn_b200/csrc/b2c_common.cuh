// Shared host/device definitions for the b2c kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include "../../include/b2c.h"

namespace b2c {

// ---- error plumbing ---------------------------------------------------------------------
void set_cuda_error(cudaError_t e, const char* where);
void count_launch();
// Programmatic dependent launch.  Every kernel of the library begins with pdl_prologue(): it waits until the
// kernel before it in the stream has completed and its writes are visible, then lets the kernel after it be
// scheduled early.  launch_pdl() marks the launch as allowed to start while its predecessor drains, so launch
// latency and the start-up of the next kernel's blocks overlap with the tail of the running one; data is only
// touched after the wait, so the stream's ordering is unchanged.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_prologue() { pdl_wait(); pdl_launch_dependents(); }

template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

inline int check_launch(const char* where) {
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_cuda_error(e, where); return B2C_ERR_CUDA; }
    return B2C_OK;
}

// ---- geometry -----------------------------------------------------------------------------
struct Geo {
    int layout, dtype, w_layout, engine;
    int n, h, w, ci, co, kh, kw, vpad, hpad, vstr, hstr, vdil, hdil;
    int ho, wo;
    int64_t M, K;   // M = n*ho*wo, K = ci*kh*kw
};

// Validate a descriptor and fill the derived fields. Output size follows
// pydtnn/layers/conv_2d.py:75-76.
inline int make_geo(const b2c_conv_desc* d, Geo& g) {
    if (!d) return B2C_ERR_NULL_POINTER;
    if (d->layout < 0 || d->layout > 1 || d->dtype < 0 || d->dtype > 1 || d->w_layout < 0 || d->w_layout > 2 ||
        d->engine < 0 || d->engine > 2)
        return B2C_ERR_BAD_ENUM;
    if (d->n <= 0 || d->h <= 0 || d->w <= 0 || d->ci <= 0 || d->co <= 0 || d->kh <= 0 || d->kw <= 0 ||
        d->vpad < 0 || d->hpad < 0 || d->vstr < 1 || d->hstr < 1 || d->vdil < 1 || d->hdil < 1)
        return B2C_ERR_BAD_GEOMETRY;
    g.layout = d->layout; g.dtype = d->dtype; g.w_layout = d->w_layout; g.engine = d->engine;
    g.n = d->n; g.h = d->h; g.w = d->w; g.ci = d->ci; g.co = d->co; g.kh = d->kh; g.kw = d->kw;
    g.vpad = d->vpad; g.hpad = d->hpad; g.vstr = d->vstr; g.hstr = d->hstr; g.vdil = d->vdil; g.hdil = d->hdil;
    int eh = d->h + 2 * d->vpad - d->vdil * (d->kh - 1) - 1;
    int ew = d->w + 2 * d->hpad - d->hdil * (d->kw - 1) - 1;
    if (eh < 0 || ew < 0) return B2C_ERR_BAD_GEOMETRY;
    g.ho = eh / d->vstr + 1;
    g.wo = ew / d->hstr + 1;
    g.M = (int64_t)g.n * g.ho * g.wo;
    g.K = (int64_t)g.ci * g.kh * g.kw;
    if (g.M > 0x7fffffffLL || g.K > 0x7fffffffLL || (int64_t)g.n * g.h * g.w > 0x7fffffffLL) return B2C_ERR_TOO_LARGE;
    return B2C_OK;
}

// Element strides of an activation tensor (n, h, w, c) in either layout.
struct ActStride { int64_t sn, sh, sw, sc; };
inline ActStride act_stride(int layout, int h, int w, int c) {
    ActStride s;
    if (layout == B2C_LAYOUT_NHWC) { s.sc = 1; s.sw = c; s.sh = (int64_t)w * c; s.sn = (int64_t)h * w * c; }
    else { s.sw = 1; s.sh = w; s.sc = (int64_t)h * w; s.sn = (int64_t)c * h * w; }
    return s;
}
// Element strides of a filter tensor by (co, ci, r, s).
struct WStride { int64_t sk, sc, sr, ss; };
inline WStride w_stride(int w_layout, int ci, int co, int kh, int kw) {
    WStride s;
    if (w_layout == B2C_W_CRSK) { s.sk = 1; s.ss = co; s.sr = (int64_t)kw * co; s.sc = (int64_t)kh * kw * co; }
    else if (w_layout == B2C_W_KCRS) { s.ss = 1; s.sr = kw; s.sc = (int64_t)kh * kw; s.sk = (int64_t)ci * kh * kw; }
    else { s.sc = 1; s.ss = ci; s.sr = (int64_t)kw * ci; s.sk = (int64_t)kh * kw * ci; }
    return s;
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ---- entry points implemented per engine ----------------------------------------------------
// generic FMA engine (conv_fma.cu)
size_t fma_workspace_bytes(const Geo& g, int pass);
int fma_fprop(const Geo& g, const void* x, const void* w, const void* bias, const b2c_bn_params* bn, int relu,
              void* y, void* ws, size_t ws_bytes, cudaStream_t st);
int fma_dgrad(const Geo& g, const void* dy, const void* w, void* dx, void* ws, size_t ws_bytes, cudaStream_t st);
int fma_wgrad(const Geo& g, const void* x, const void* dy, void* dw, void* db, void* ws, size_t ws_bytes,
              cudaStream_t st);
int fma_index_map(const Geo& g, int64_t* map, cudaStream_t st);
int channel_sum(int dtype, int layout, int n, int c, int hw, const void* src, void* dst, void* ws, size_t ws_bytes,
                cudaStream_t st);
size_t channel_sum_workspace_bytes(int n, int c, int hw);
int channel_sum_v4(int n, int c, int hw, const void* src, void* dst, void* ws, size_t ws_bytes, cudaStream_t st);

// tensor-core engine (conv_tc.cu)
bool tc_supported(const Geo& g, int pass);
int tc_wait_selftest(long long limit_cycles, cudaStream_t st);
size_t tc_workspace_bytes(const Geo& g, int pass);
int tc_fprop(const Geo& g, const void* x, const void* w, const void* bias, const b2c_bn_params* bn, int relu,
             void* y, void* ws, size_t ws_bytes, cudaStream_t st);
int tc_dgrad(const Geo& g, const void* dy, const void* w, void* dx, void* ws, size_t ws_bytes, cudaStream_t st);
int tc_wgrad(const Geo& g, const void* x, const void* dy, void* dw, void* db, void* ws, size_t ws_bytes,
             cudaStream_t st);
int tc_read_status(int* out);
bool tc_keeps_lowered(const Geo& g);
int tc_wgrad_lowered(const Geo& g, const void* x, const void* dy, void* dw, void* db, void* ws, size_t ws_bytes, cudaStream_t st);
bool tc_fc_small_batch(int dtype, int engine, int batch, int in_f, int out_f);
size_t tc_fc_small_batch_bytes(int batch, int in_f, int out_f);
int tc_fc_forward_small_batch(int batch, int in_f, int out_f, const void* x, const void* w, const void* bias, void* y,
                              void* ws, size_t ws_bytes, cudaStream_t st);
int tc_fc_dgrad_small_batch(int batch, int in_f, int out_f, const void* dy, const void* w, void* dx, void* ws, size_t ws_bytes, cudaStream_t st);
int tc_fc_wgrad_small_batch(int batch, int in_f, int out_f, const void* x, const void* dy, void* dw, void* db, void* ws, size_t ws_bytes,
                            cudaStream_t st);
size_t tc_stats_bytes(const Geo& g);
int tc_fprop_stats(const Geo& g, const void* x, const void* w, const void* bias, void* y, void* stats, size_t stats_bytes,
                   void* ws, size_t ws_bytes, cudaStream_t st);

}  // namespace b2c

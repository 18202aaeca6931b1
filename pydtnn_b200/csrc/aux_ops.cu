// HBM-bound layers either side of the convolution in a training step: batch normalisation,
// ReLU, residual sum, pooling, softmax, categorical cross-entropy and SGD.  All are single-pass
// streaming kernels over NHWC (rows, c) or NCHW (n, c, hw) tensors; per-channel reductions are
// two-stage with double partial sums so the result does not depend on launch order.
#include "b2c_common.cuh"
#include <float.h>
#include <mutex>

namespace b2c {

#define RED_CHUNKS 64

// ---- two-value per-channel reduction ---------------------------------------------------------
// F(flat_index, channel) -> (v0, v1); partial[chunk][2][c] in double.
template <typename F>
__global__ void reduce2_nhwc_kernel(F f, double* __restrict__ partial, int64_t rows, int c)
{
    pdl_prologue();
    __shared__ double s0[8][33], s1[8][33];
    int ch = blockIdx.x * 32 + threadIdx.x;
    int64_t per = (rows + gridDim.y - 1) / gridDim.y;
    int64_t r0 = (int64_t)blockIdx.y * per, r1 = r0 + per < rows ? r0 + per : rows;
    double a0 = 0.0, a1 = 0.0;
    if (ch < c)
        for (int64_t r = r0 + threadIdx.y; r < r1; r += 8) { double v0, v1; f(r * c + ch, ch, v0, v1); a0 += v0; a1 += v1; }
    s0[threadIdx.y][threadIdx.x] = a0; s1[threadIdx.y][threadIdx.x] = a1;
    __syncthreads();
    if (threadIdx.y == 0 && ch < c) {
        double t0 = 0.0, t1 = 0.0;
        for (int i = 0; i < 8; i++) { t0 += s0[i][threadIdx.x]; t1 += s1[i][threadIdx.x]; }
        partial[((int64_t)blockIdx.y * 2 + 0) * c + ch] = t0;
        partial[((int64_t)blockIdx.y * 2 + 1) * c + ch] = t1;
    }
}

template <typename F>
__global__ void reduce2_nchw_kernel(F f, double* __restrict__ partial, int n, int c, int hw)
{
    pdl_prologue();
    __shared__ double s0[256], s1[256];
    int ch = blockIdx.x;
    int64_t total = (int64_t)n * hw;
    int64_t per = (total + gridDim.y - 1) / gridDim.y;
    int64_t i0 = (int64_t)blockIdx.y * per, i1 = i0 + per < total ? i0 + per : total;
    double a0 = 0.0, a1 = 0.0;
    for (int64_t i = i0 + threadIdx.x; i < i1; i += 256) {
        int64_t img = i / hw, pos = i - img * hw;
        double v0, v1; f((img * c + ch) * hw + pos, ch, v0, v1); a0 += v0; a1 += v1;
    }
    s0[threadIdx.x] = a0; s1[threadIdx.x] = a1;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if (threadIdx.x < s) { s0[threadIdx.x] += s0[threadIdx.x + s]; s1[threadIdx.x] += s1[threadIdx.x + s]; }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        partial[((int64_t)blockIdx.y * 2 + 0) * c + ch] = s0[0];
        partial[((int64_t)blockIdx.y * 2 + 1) * c + ch] = s1[0];
    }
}

template <typename F>
static int launch_reduce2(F f, double* partial, int layout, int n, int c, int hw, int& chunks, cudaStream_t st)
{
    int64_t rows = (int64_t)n * hw;
    chunks = (int)(rows < RED_CHUNKS ? rows : RED_CHUNKS);
    if (chunks < 1) chunks = 1;
    if (layout == B2C_LAYOUT_NHWC) {
        dim3 grid((c + 31) / 32, chunks), block(32, 8);
        launch_pdl(reduce2_nhwc_kernel<F>, grid, block, 0, st, f, partial, rows, c);
    } else {
        dim3 grid(c, chunks);
        launch_pdl(reduce2_nchw_kernel<F>, grid, 256, 0, st, f, partial, n, c, hw);
    }
    return check_launch("reduce2");
}

static size_t reduce2_bytes(int c) { return (size_t)RED_CHUNKS * 2 * c * sizeof(double); }

__device__ __forceinline__ int channel_of(int64_t idx, int c, int hw, int nchw)
{
    return nchw ? (int)((idx / hw) % c) : (int)(idx % c);
}

// ---- batch normalisation ---------------------------------------------------------------------

template <typename T> struct StatF {
    const T* x;
    __device__ void operator()(int64_t i, int, double& v0, double& v1) const { double v = (double)x[i]; v0 = v; v1 = v * v; }
};

template <typename T>
__global__ void bn_stats_final_kernel(const double* __restrict__ partial, int chunks, int c, double count,
                                      double momentum, double eps, T* running_mean, T* running_var,
                                      T* save_mean, T* save_inv_std)
{
    pdl_prologue();
    int ch = blockIdx.x * blockDim.x + threadIdx.x;
    if (ch >= c) return;
    double s = 0.0, ss = 0.0;
    for (int i = 0; i < chunks; i++) { s += partial[((int64_t)i * 2) * c + ch]; ss += partial[((int64_t)i * 2 + 1) * c + ch]; }
    double mean = s / count;
    double var = ss / count - mean * mean;
    if (var < 0.0) var = 0.0;
    save_mean[ch] = (T)mean;
    save_inv_std[ch] = (T)(1.0 / sqrt(var + eps));
    running_mean[ch] = (T)(momentum * (double)running_mean[ch] + (1.0 - momentum) * mean);
    running_var[ch] = (T)(momentum * (double)running_var[ch] + (1.0 - momentum) * var);
}

template <typename T>
__global__ void bn_apply_kernel(const T* __restrict__ x, T* __restrict__ y, const T* __restrict__ mean,
                                const T* __restrict__ inv_std, const T* __restrict__ gamma, const T* __restrict__ beta,
                                int64_t total, int c, int hw, int nchw, int relu, int ref_order, const T* __restrict__ addend)
{
    pdl_prologue();
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        int ch = channel_of(i, c, hw, nchw);
        T xn = (x[i] - mean[ch]) * inv_std[ch];
        T v = ref_order ? (xn * gamma[ch] + beta[ch]) : (gamma[ch] * xn + beta[ch]);
        if (addend) v = v + addend[i];        // residual sum: the rounded BN output plus the other branch
        if (relu) v = v > T(0) ? v : T(0);
        y[i] = v;
    }
}

template <typename T> struct BnBwdF {
    const T *x, *dy, *y, *mean, *inv_std; int relu;
    __device__ void operator()(int64_t i, int ch, double& v0, double& v1) const {
        T g = dy[i];
        if (relu && !(y[i] > T(0))) g = T(0);
        T xn = (x[i] - mean[ch]) * inv_std[ch];
        v0 = (double)g * (double)xn; v1 = (double)g;
    }
};

template <typename T>
__global__ void bn_bwd_final_kernel(const double* __restrict__ partial, int chunks, int c, T* dgamma, T* dbeta)
{
    pdl_prologue();
    int ch = blockIdx.x * blockDim.x + threadIdx.x;
    if (ch >= c) return;
    double s0 = 0.0, s1 = 0.0;
    for (int i = 0; i < chunks; i++) { s0 += partial[((int64_t)i * 2) * c + ch]; s1 += partial[((int64_t)i * 2 + 1) * c + ch]; }
    dgamma[ch] = (T)s0; dbeta[ch] = (T)s1;
}

// dx = (gamma / (std*n)) * (n*dy - xn*dgamma - dbeta)   (pydtnn/cython_modules/bn_training_cython.pyx:227)
template <typename T>
__global__ void bn_bwd_dx_kernel(const T* __restrict__ x, const T* __restrict__ dy, const T* __restrict__ y,
                                 const T* __restrict__ gamma, const T* __restrict__ mean, const T* __restrict__ inv_std,
                                 const T* __restrict__ dgamma, const T* __restrict__ dbeta, T* __restrict__ dx,
                                 int64_t total, int c, int hw, int nchw, int relu, T count)
{
    pdl_prologue();
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        int ch = channel_of(i, c, hw, nchw);
        T g = dy[i];
        if (relu && !(y[i] > T(0))) g = T(0);
        T xn = (x[i] - mean[ch]) * inv_std[ch];
        dx[i] = (gamma[ch] * inv_std[ch] / count) * (count * g - xn * dgamma[ch] - dbeta[ch]);
    }
}


// ---- float32 NHWC fast path (c % 4 == 0): float4 loads, per-thread fixed channel group ----------
// The tensor is (rows, c4) float4 with c4 = c/4. A block is RX x CX threads (CX = min(c4, 64) channel
// groups, RX = 256 / CX row lanes); grid.x walks channel-group blocks, grid.y row chunks. Every
// thread keeps its 4 channels, so per-channel parameters are loaded once and reductions need no
// index arithmetic per element.
struct V4Geo { int c4, cx, rx, gx, chunks; int64_t rows; };

static bool v4_ok(int dtype, int layout, int c, const void* a, const void* b, const void* d)
{
    if (dtype != B2C_F32 || layout != B2C_LAYOUT_NHWC || c % 4) return false;
    int c4 = c / 4;
    int cx = c4 < 64 ? c4 : 64;
    if (256 % cx || c4 % cx) return false;
    return (((uintptr_t)a | (uintptr_t)b | (uintptr_t)d) & 15) == 0;
}
static V4Geo v4_geo(int64_t rows, int c, int max_chunks)
{
    V4Geo g; g.c4 = c / 4; g.cx = g.c4 < 64 ? g.c4 : 64; g.rx = 256 / g.cx; g.gx = g.c4 / g.cx; g.rows = rows;
    int64_t want = (148 * 4 + g.gx - 1) / g.gx;
    int64_t by_rows = (rows + g.rx * 4 - 1) / (g.rx * 4);          // at least 4 rows per thread
    int64_t ch = want < by_rows ? want : by_rows;
    if (ch > max_chunks) ch = max_chunks;
    if (ch < 1) ch = 1;
    g.chunks = (int)ch;
    return g;
}

// F(float4 index, channel-group index, v0[4], v1[4]) ; partial[chunk][2][c] doubles
template <typename F>
__global__ void __launch_bounds__(256) reduce2_v4_kernel(F f, double* __restrict__ partial, V4Geo g)
{
    pdl_prologue();
    __shared__ float sm[256][9];
    const int cxi = threadIdx.x % g.cx, rxi = threadIdx.x / g.cx;
    const int grp = blockIdx.x * g.cx + cxi;
    const int64_t per = (g.rows + gridDim.y - 1) / gridDim.y;
    // Blocks start in index order; the first ones take the *last* rows. The tensor was just written front to back
    // by the kernel before, so its tail is what L2 still holds, and the pass that follows this one (apply / dx)
    // walks front to back and finds the rows this pass read last.
    const int chunk = gridDim.y - 1 - blockIdx.y;
    const int64_t r0 = (int64_t)chunk * per, r1 = r0 + per < g.rows ? r0 + per : g.rows;
    float a0[4] = {0.f, 0.f, 0.f, 0.f}, a1[4] = {0.f, 0.f, 0.f, 0.f};
    int64_t r = r0 + rxi;
    if (F::UNROLL > 1) {
        // several rows per trip, their loads issued together; the additions keep the row order
        constexpr int U = F::UNROLL;
        for (; r + (U - 1) * (int64_t)g.rx < r1; r += U * (int64_t)g.rx) {
            float v0[U][4], v1[U][4];
#pragma unroll
            for (int u = 0; u < U; u++) f((r + u * (int64_t)g.rx) * g.c4 + grp, grp, v0[u], v1[u]);
#pragma unroll
            for (int u = 0; u < U; u++)
#pragma unroll
                for (int e = 0; e < 4; e++) { a0[e] += v0[u][e]; a1[e] += v1[u][e]; }
        }
    }
    for (; r < r1; r += g.rx) {
        float v0[4], v1[4];
        f(r * g.c4 + grp, grp, v0, v1);
#pragma unroll
        for (int e = 0; e < 4; e++) { a0[e] += v0[e]; a1[e] += v1[e]; }
    }
#pragma unroll
    for (int e = 0; e < 4; e++) { sm[threadIdx.x][e] = a0[e]; sm[threadIdx.x][4 + e] = a1[e]; }
    __syncthreads();
    if (rxi == 0) {
        double t[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int i = 0; i < g.rx; i++)
#pragma unroll
            for (int e = 0; e < 8; e++) t[e] += (double)sm[i * g.cx + cxi][e];
        const int c = g.c4 * 4;
#pragma unroll
        for (int e = 0; e < 4; e++) {
            partial[((int64_t)chunk * 2 + 0) * c + grp * 4 + e] = t[e];
            partial[((int64_t)chunk * 2 + 1) * c + grp * 4 + e] = t[4 + e];
        }
    }
}

// The batch-norm output before the ReLU, in one fixed instruction sequence: the forward kernel stores
// max(bn_affine(..), 0) and the backward kernels recompute bn_affine(..) > 0 as the ReLU mask from x instead of
// reading y back, so both must round identically.
__device__ __forceinline__ float bn_affine(float v, float m, float is, float ga, float be)
{
    return __fmaf_rn(ga, __fmul_rn(__fsub_rn(v, m), is), be);
}

struct StatV4 {
    static constexpr int UNROLL = 4;
    const float4* x;
    __device__ void operator()(int64_t j, int, float (&v0)[4], float (&v1)[4]) const {
        float4 v = x[j];
        v0[0] = v.x; v0[1] = v.y; v0[2] = v.z; v0[3] = v.w;
        v1[0] = v.x * v.x; v1[1] = v.y * v.y; v1[2] = v.z * v.z; v1[3] = v.w * v.w;
    }
};
struct SumV4 {   // plain per-channel sum (bias gradient)
    static constexpr int UNROLL = 4;
    const float4* x;
    __device__ void operator()(int64_t j, int, float (&v0)[4], float (&v1)[4]) const {
        float4 v = x[j];
        v0[0] = v.x; v0[1] = v.y; v0[2] = v.z; v0[3] = v.w;
        v1[0] = v1[1] = v1[2] = v1[3] = 0.f;
    }
};
struct BnBwdV4 {
    static constexpr int UNROLL = 1;      // two and four rows per trip were measured: no faster (more registers, fewer resident blocks)
    const float4 *x, *dy, *y; const float *mean, *inv_std, *gamma, *beta; int relu;     // beta != null: mask from x
    __device__ void operator()(int64_t j, int grp, float (&v0)[4], float (&v1)[4]) const {
        float4 xv = x[j], g = dy[j];
        const float4 m = *reinterpret_cast<const float4*>(mean + grp * 4), is = *reinterpret_cast<const float4*>(inv_std + grp * 4);
        if (relu) {
            if (beta) {
                const float4 ga = *reinterpret_cast<const float4*>(gamma + grp * 4), be = *reinterpret_cast<const float4*>(beta + grp * 4);
                if (!(bn_affine(xv.x, m.x, is.x, ga.x, be.x) > 0.f)) g.x = 0.f;
                if (!(bn_affine(xv.y, m.y, is.y, ga.y, be.y) > 0.f)) g.y = 0.f;
                if (!(bn_affine(xv.z, m.z, is.z, ga.z, be.z) > 0.f)) g.z = 0.f;
                if (!(bn_affine(xv.w, m.w, is.w, ga.w, be.w) > 0.f)) g.w = 0.f;
            } else {
                float4 yv = y[j]; if (!(yv.x > 0.f)) g.x = 0.f; if (!(yv.y > 0.f)) g.y = 0.f; if (!(yv.z > 0.f)) g.z = 0.f; if (!(yv.w > 0.f)) g.w = 0.f;
            }
        }
        v0[0] = g.x * ((xv.x - m.x) * is.x); v0[1] = g.y * ((xv.y - m.y) * is.y);
        v0[2] = g.z * ((xv.z - m.z) * is.z); v0[3] = g.w * ((xv.w - m.w) * is.w);
        v1[0] = g.x; v1[1] = g.y; v1[2] = g.z; v1[3] = g.w;
    }
};

// Four warps per channel sum the per-chunk partials: every thread adds its chunks (128 apart) in index order, a shuffle
// tree adds the lanes of a warp, and the four warp sums are added in warp order -- a fixed order whatever the launch.
// With a few hundred chunks a thread has a handful of independent loads, so the kernel costs one memory round trip.
// mode 0: batch statistics -> save_mean, save_inv_std, running averages. mode 1: (dgamma, dbeta).
// mode 2: single sum -> out0.
__global__ void __launch_bounds__(256) reduce2_final_warp_kernel(const double* __restrict__ partial, int chunks, int c, int mode, double count,
                                                                 double momentum, double eps, float* out0, float* out1, float* run0, float* run1)
{
    pdl_prologue();
    __shared__ double w0[2][4], w1[2][4];
    const int sub = threadIdx.x >> 7;                       // which of the block's two channels
    const int ch = blockIdx.x * 2 + sub;
    const int t = threadIdx.x & 127, lane = threadIdx.x & 31, wrp = t >> 5;
    double s0 = 0.0, s1 = 0.0;
    if (ch < c) {
        int i = t;
        for (; i + 384 < chunks; i += 512) {
            double a0[4], a1[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                a0[u] = partial[((int64_t)(i + 128 * u) * 2) * c + ch];
                a1[u] = partial[((int64_t)(i + 128 * u) * 2 + 1) * c + ch];
            }
#pragma unroll
            for (int u = 0; u < 4; u++) { s0 += a0[u]; s1 += a1[u]; }
        }
        for (; i < chunks; i += 128) { s0 += partial[((int64_t)i * 2) * c + ch]; s1 += partial[((int64_t)i * 2 + 1) * c + ch]; }
    }
    for (int o = 16; o > 0; o >>= 1) { s0 += __shfl_down_sync(0xffffffffu, s0, o); s1 += __shfl_down_sync(0xffffffffu, s1, o); }
    if (lane == 0) { w0[sub][wrp] = s0; w1[sub][wrp] = s1; }
    __syncthreads();
    if (t != 0 || ch >= c) return;
    s0 = ((w0[sub][0] + w0[sub][1]) + w0[sub][2]) + w0[sub][3];
    s1 = ((w1[sub][0] + w1[sub][1]) + w1[sub][2]) + w1[sub][3];
    if (mode == 0) {
        double mean = s0 / count, var = s1 / count - mean * mean;
        if (var < 0.0) var = 0.0;
        out0[ch] = (float)mean; out1[ch] = (float)(1.0 / sqrt(var + eps));
        run0[ch] = (float)(momentum * (double)run0[ch] + (1.0 - momentum) * mean);
        run1[ch] = (float)(momentum * (double)run1[ch] + (1.0 - momentum) * var);
    } else if (mode == 1) { out0[ch] = (float)s0; out1[ch] = (float)s1; }
    else out0[ch] = (float)s0;
}

__global__ void __launch_bounds__(256) bn_apply_v4_kernel(const float4* __restrict__ x, float4* __restrict__ y, const float* __restrict__ mean,
                                                          const float* __restrict__ inv_std, const float* __restrict__ gamma,
                                                          const float* __restrict__ beta, V4Geo g, int relu,
                                                          const float4* __restrict__ addend)
{
    pdl_prologue();
    const int cxi = threadIdx.x % g.cx, rxi = threadIdx.x / g.cx;
    const int grp = blockIdx.x * g.cx + cxi;
    const float4 m = *reinterpret_cast<const float4*>(mean + grp * 4), is = *reinterpret_cast<const float4*>(inv_std + grp * 4);
    const float4 ga = *reinterpret_cast<const float4*>(gamma + grp * 4), be = *reinterpret_cast<const float4*>(beta + grp * 4);
    const int64_t per = (g.rows + gridDim.y - 1) / gridDim.y;
    const int64_t r0 = (int64_t)blockIdx.y * per, r1 = r0 + per < g.rows ? r0 + per : g.rows;
    auto one = [&](float4 v, float4 a) {
        float4 o;
        o.x = bn_affine(v.x, m.x, is.x, ga.x, be.x); o.y = bn_affine(v.y, m.y, is.y, ga.y, be.y);
        o.z = bn_affine(v.z, m.z, is.z, ga.z, be.z); o.w = bn_affine(v.w, m.w, is.w, ga.w, be.w);
        if (addend) {        // residual sum on the rounded BN output, as the separate add kernel would do
            o.x = __fadd_rn(o.x, a.x); o.y = __fadd_rn(o.y, a.y); o.z = __fadd_rn(o.z, a.z); o.w = __fadd_rn(o.w, a.w);
        }
        if (relu) { o.x = fmaxf(o.x, 0.f); o.y = fmaxf(o.y, 0.f); o.z = fmaxf(o.z, 0.f); o.w = fmaxf(o.w, 0.f); }
        return o;
    };
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    int64_t r = r0 + rxi;
    for (; r + g.rx < r1; r += 2 * g.rx) {          // two rows per trip: their loads are in flight together
        const int64_t j0 = r * g.c4 + grp, j1 = (r + g.rx) * g.c4 + grp;
        const float4 v0 = x[j0], v1 = x[j1];
        const float4 a0 = addend ? addend[j0] : zero, a1 = addend ? addend[j1] : zero;
        y[j0] = one(v0, a0); y[j1] = one(v1, a1);
    }
    if (r < r1) {
        const int64_t j = r * g.c4 + grp;
        y[j] = one(x[j], addend ? addend[j] : zero);
    }
}

__global__ void __launch_bounds__(256) bn_bwd_dx_v4_kernel(const float4* __restrict__ x, const float4* __restrict__ dy, const float4* __restrict__ y,
                                                           const float* __restrict__ gamma, const float* __restrict__ mean,
                                                           const float* __restrict__ inv_std, const float* __restrict__ dgamma,
                                                           const float* __restrict__ dbeta, float4* __restrict__ dx, V4Geo g, int relu, float count,
                                                           const float* __restrict__ beta)
{
    pdl_prologue();
    const int cxi = threadIdx.x % g.cx, rxi = threadIdx.x / g.cx;
    const int grp = blockIdx.x * g.cx + cxi;
    const float4 m = *reinterpret_cast<const float4*>(mean + grp * 4), is = *reinterpret_cast<const float4*>(inv_std + grp * 4);
    const float4 ga = *reinterpret_cast<const float4*>(gamma + grp * 4);
    const float4 dg = *reinterpret_cast<const float4*>(dgamma + grp * 4), db = *reinterpret_cast<const float4*>(dbeta + grp * 4);
    const float4 sc = make_float4(ga.x * is.x / count, ga.y * is.y / count, ga.z * is.z / count, ga.w * is.w / count);
    const int64_t per = (g.rows + gridDim.y - 1) / gridDim.y;
    const int64_t r0 = (int64_t)blockIdx.y * per, r1 = r0 + per < g.rows ? r0 + per : g.rows;
    const float4 be = (relu && beta) ? *reinterpret_cast<const float4*>(beta + grp * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    auto one = [&](int64_t j, float4 xv, float4 gd) {
        float4 o;
        if (relu && beta) {       // ReLU mask recomputed from x (see bn_affine)
            if (!(bn_affine(xv.x, m.x, is.x, ga.x, be.x) > 0.f)) gd.x = 0.f;
            if (!(bn_affine(xv.y, m.y, is.y, ga.y, be.y) > 0.f)) gd.y = 0.f;
            if (!(bn_affine(xv.z, m.z, is.z, ga.z, be.z) > 0.f)) gd.z = 0.f;
            if (!(bn_affine(xv.w, m.w, is.w, ga.w, be.w) > 0.f)) gd.w = 0.f;
        } else if (relu) { float4 yv = y[j]; if (!(yv.x > 0.f)) gd.x = 0.f; if (!(yv.y > 0.f)) gd.y = 0.f; if (!(yv.z > 0.f)) gd.z = 0.f; if (!(yv.w > 0.f)) gd.w = 0.f; }
        o.x = sc.x * (count * gd.x - ((xv.x - m.x) * is.x) * dg.x - db.x);
        o.y = sc.y * (count * gd.y - ((xv.y - m.y) * is.y) * dg.y - db.y);
        o.z = sc.z * (count * gd.z - ((xv.z - m.z) * is.z) * dg.z - db.z);
        o.w = sc.w * (count * gd.w - ((xv.w - m.w) * is.w) * dg.w - db.w);
        return o;
    };
    int64_t r = r0 + rxi;
    for (; r + g.rx < r1; r += 2 * g.rx) {          // two rows per trip: their loads are in flight together
        const int64_t j0 = r * g.c4 + grp, j1 = (r + g.rx) * g.c4 + grp;
        const float4 x0 = x[j0], g0 = dy[j0], x1 = x[j1], g1 = dy[j1];
        dx[j0] = one(j0, x0, g0); dx[j1] = one(j1, x1, g1);
    }
    if (r < r1) {
        const int64_t j = r * g.c4 + grp;
        dx[j] = one(j, x[j], dy[j]);
    }
}

// First stage of the batch statistics from the partial sums a convolution left while it stored its output
// (conv_tc.cu): `sums` = [rows][2][c] floats, one row per 32 output rows.  Block (32 channels, 8 row lanes), grid
// (c / 32, chunks): a thread adds the rows of its chunk, 8 apart, in index order in double; the 8 row lanes are added
// in lane order; result partial[chunk][2][c] in double, the input format of reduce2_final_warp_kernel.
__global__ void __launch_bounds__(256) bn_conv_sums_kernel(const float* __restrict__ sums, int rows, int c, double* __restrict__ partial)
{
    pdl_prologue();
    __shared__ double s0[8][33], s1[8][33];
    const int ch = blockIdx.x * 32 + threadIdx.x;
    const int per = (rows + gridDim.y - 1) / gridDim.y;
    const int r0 = blockIdx.y * per, r1 = r0 + per < rows ? r0 + per : rows;
    double a0 = 0.0, a1 = 0.0;
    if (ch < c) {
        int i = r0 + threadIdx.y;
        for (; i + 24 < r1; i += 32) {          // four independent row pairs in flight, added in index order
            float u0[4], u1[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                u0[u] = __ldcg(sums + ((size_t)(i + 8 * u) * 2) * c + ch);
                u1[u] = __ldcg(sums + ((size_t)(i + 8 * u) * 2 + 1) * c + ch);
            }
#pragma unroll
            for (int u = 0; u < 4; u++) { a0 += (double)u0[u]; a1 += (double)u1[u]; }
        }
        for (; i < r1; i += 8) {
            a0 += (double)__ldcg(sums + ((size_t)i * 2) * c + ch);
            a1 += (double)__ldcg(sums + ((size_t)i * 2 + 1) * c + ch);
        }
    }
    s0[threadIdx.y][threadIdx.x] = a0; s1[threadIdx.y][threadIdx.x] = a1;
    __syncthreads();
    if (threadIdx.y == 0 && ch < c) {
        double t0 = 0.0, t1 = 0.0;
        for (int i = 0; i < 8; i++) { t0 += s0[i][threadIdx.x]; t1 += s1[i][threadIdx.x]; }
        partial[((size_t)blockIdx.y * 2 + 0) * c + ch] = t0;
        partial[((size_t)blockIdx.y * 2 + 1) * c + ch] = t1;
    }
}

// The batch statistics from a few rows of partial sums (a convolution that kept one row per CTA group): block
// (32 channels, 32 row lanes), one block per 32 channels.  A thread adds its rows (32 apart) in index order in double,
// the 32 row lanes are added in lane order, then mean, inverse deviation and the running averages as
// reduce2_final_warp_kernel (mode 0) writes them.
__global__ void __launch_bounds__(1024) bn_rows_final_kernel(const float* __restrict__ sums, int rows, int c, double count, double momentum,
                                                             double eps, float* __restrict__ mean_out, float* __restrict__ inv_std_out,
                                                             float* __restrict__ run_mean, float* __restrict__ run_var)
{
    pdl_prologue();
    __shared__ double s0[32][33], s1[32][33];
    const int ch = blockIdx.x * 32 + threadIdx.x;
    double a0 = 0.0, a1 = 0.0;
    if (ch < c) {
        int i = threadIdx.y;
        for (; i + 96 < rows; i += 128) {        // four independent row pairs in flight, added in index order
            float u0[4], u1[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                u0[u] = __ldcg(sums + ((size_t)(i + 32 * u) * 2) * c + ch);
                u1[u] = __ldcg(sums + ((size_t)(i + 32 * u) * 2 + 1) * c + ch);
            }
#pragma unroll
            for (int u = 0; u < 4; u++) { a0 += (double)u0[u]; a1 += (double)u1[u]; }
        }
        for (; i < rows; i += 32) {
            a0 += (double)__ldcg(sums + ((size_t)i * 2) * c + ch);
            a1 += (double)__ldcg(sums + ((size_t)i * 2 + 1) * c + ch);
        }
    }
    s0[threadIdx.y][threadIdx.x] = a0; s1[threadIdx.y][threadIdx.x] = a1;
    __syncthreads();
    if (threadIdx.y != 0 || ch >= c) return;
    double t0 = 0.0, t1 = 0.0;
    for (int i = 0; i < 32; i++) { t0 += s0[i][threadIdx.x]; t1 += s1[i][threadIdx.x]; }
    double mean = t0 / count, var = t1 / count - mean * mean;
    if (var < 0.0) var = 0.0;
    mean_out[ch] = (float)mean; inv_std_out[ch] = (float)(1.0 / sqrt(var + eps));
    run_mean[ch] = (float)(momentum * (double)run_mean[ch] + (1.0 - momentum) * mean);
    run_var[ch] = (float)(momentum * (double)run_var[ch] + (1.0 - momentum) * var);
}

static V4Geo v4_apply_geo(int64_t rows, int c)
{
    V4Geo g = v4_geo(rows, c, 1 << 20);
    int64_t want = (148 * 8 + g.gx - 1) / g.gx;
    int64_t by_rows = (rows + g.rx * 4 - 1) / (g.rx * 4);
    g.chunks = (int)(want < by_rows ? want : by_rows);
    if (g.chunks < 1) g.chunks = 1;
    return g;
}

static int final_warp(const double* partial, int chunks, int c, int mode, double count, double momentum, double eps,
                      float* o0, float* o1, float* r0, float* r1, cudaStream_t st)
{
    launch_pdl(reduce2_final_warp_kernel, (c + 1) / 2, 256, 0, st, partial, chunks, c, mode, count, momentum, eps, o0, o1, r0, r1);
    return check_launch("reduce2_final_warp");
}

// Per-channel sum of an NHWC float32 tensor through the fast path (used for the bias gradient).
int channel_sum_v4(int n, int c, int hw, const void* src, void* dst, void* ws, size_t ws_bytes, cudaStream_t st)
{
    if (!v4_ok(B2C_F32, B2C_LAYOUT_NHWC, c, src, src, src)) return 1;   // not applicable
    int max_chunks = (int)(ws_bytes / ((size_t)2 * c * sizeof(double)));
    if (max_chunks < 1) return 1;
    V4Geo g = v4_geo((int64_t)n * hw, c, max_chunks);
    SumV4 f{(const float4*)src};
    launch_pdl(reduce2_v4_kernel<SumV4>, dim3(g.gx, g.chunks), 256, 0, st, f, (double*)ws, g);
    int rc = check_launch("reduce2_v4(sum)"); if (rc) return rc;
    return final_warp((const double*)ws, g.chunks, c, 2, 1.0, 0.0, 0.0, (float*)dst, nullptr, nullptr, nullptr, st);
}

static unsigned ew_blocks(int64_t total) { int64_t b = (total + 255) / 256; return (unsigned)(b > 148 * 16 ? 148 * 16 : (b < 1 ? 1 : b)); }

template <typename T>
static int bn_train_forward_t(int layout, int n, int c, int hw, const T* x, const T* gamma, const T* beta,
                              T* rm, T* rv, double momentum, double eps, int relu, T* y, T* sm, T* si,
                              double* scratch, size_t scratch_bytes, cudaStream_t st, const T* addend = nullptr)
{
    if (sizeof(T) == 4 && v4_ok(B2C_F32, layout, c, x, y, addend ? (const void*)addend : (const void*)x)) {
        int max_chunks = (int)(scratch_bytes / ((size_t)2 * c * sizeof(double)));
        V4Geo g = v4_geo((int64_t)n * hw, c, max_chunks);
        StatV4 f{(const float4*)x};
        launch_pdl(reduce2_v4_kernel<StatV4>, dim3(g.gx, g.chunks), 256, 0, st, f, scratch, g);
        int rc = check_launch("reduce2_v4(stats)"); if (rc) return rc;
        rc = final_warp(scratch, g.chunks, c, 0, (double)n * hw, momentum, eps, (float*)sm, (float*)si, (float*)rm, (float*)rv, st);
        if (rc) return rc;
        V4Geo ga = v4_apply_geo((int64_t)n * hw, c);
        launch_pdl(bn_apply_v4_kernel, dim3(ga.gx, ga.chunks), 256, 0, st, (const float4*)x, (float4*)y, (const float*)sm, (const float*)si,
                                                                  (const float*)gamma, (const float*)beta, ga, relu, (const float4*)addend);
        return check_launch("bn_apply_v4");
    }
    int chunks;
    StatF<T> f{x};
    int rc = launch_reduce2(f, scratch, layout, n, c, hw, chunks, st);
    if (rc) return rc;
    launch_pdl(bn_stats_final_kernel<T>, (c + 127) / 128, 128, 0, st, scratch, chunks, c, (double)n * hw, momentum, eps, rm, rv, sm, si);
    rc = check_launch("bn_stats_final"); if (rc) return rc;
    int64_t total = (int64_t)n * c * hw;
    launch_pdl(bn_apply_kernel<T>, ew_blocks(total), 256, 0, st, x, y, sm, si, gamma, beta, total, c, hw, layout == B2C_LAYOUT_NCHW, relu, 0, addend);
    return check_launch("bn_apply");
}

template <typename T>
static int bn_train_backward_t(int layout, int n, int c, int hw, const T* x, const T* dy, const T* y, const T* beta, const T* gamma,
                               const T* sm, const T* si, T* dgamma, T* dbeta, T* dx, double* scratch, size_t scratch_bytes,
                               cudaStream_t st)
{
    int chunks;
    int relu = y != nullptr || beta != nullptr;
    if (sizeof(T) == 4 && v4_ok(B2C_F32, layout, c, x, dy, dx ? (const void*)dx : (const void*)x) && (beta || !y || ((uintptr_t)y & 15) == 0)) {
        int max_chunks = (int)(scratch_bytes / ((size_t)2 * c * sizeof(double)));
        V4Geo g = v4_geo((int64_t)n * hw, c, max_chunks);
        BnBwdV4 f{(const float4*)x, (const float4*)dy, (const float4*)y, (const float*)sm, (const float*)si, (const float*)gamma,
                  (const float*)beta, relu};
        launch_pdl(reduce2_v4_kernel<BnBwdV4>, dim3(g.gx, g.chunks), 256, 0, st, f, scratch, g);
        int rc = check_launch("reduce2_v4(bn_bwd)"); if (rc) return rc;
        rc = final_warp(scratch, g.chunks, c, 1, 1.0, 0.0, 0.0, (float*)dgamma, (float*)dbeta, nullptr, nullptr, st);
        if (rc || !dx) return rc;
        V4Geo ga = v4_apply_geo((int64_t)n * hw, c);
        launch_pdl(bn_bwd_dx_v4_kernel, dim3(ga.gx, ga.chunks), 256, 0, st, (const float4*)x, (const float4*)dy, (const float4*)y, (const float*)gamma,
                                                                   (const float*)sm, (const float*)si, (const float*)dgamma, (const float*)dbeta,
                                                                   (float4*)dx, ga, relu, (float)((double)n * hw), (const float*)beta);
        return check_launch("bn_bwd_dx_v4");
    }
    if (relu && !y) return B2C_ERR_NULL_POINTER;        // this path reads the mask from y
    BnBwdF<T> f{x, dy, y, sm, si, relu};
    int rc = launch_reduce2(f, scratch, layout, n, c, hw, chunks, st);
    if (rc) return rc;
    launch_pdl(bn_bwd_final_kernel<T>, (c + 127) / 128, 128, 0, st, scratch, chunks, c, dgamma, dbeta);
    rc = check_launch("bn_bwd_final"); if (rc) return rc;
    if (!dx) return B2C_OK;
    int64_t total = (int64_t)n * c * hw;
    launch_pdl(bn_bwd_dx_kernel<T>, ew_blocks(total), 256, 0, st, x, dy, y, gamma, sm, si, dgamma, dbeta, dx, total, c, hw,
                                                          layout == B2C_LAYOUT_NCHW, relu, (T)((double)n * hw));
    return check_launch("bn_bwd_dx");
}

// ---- elementwise ---------------------------------------------------------------------------

template <typename T> __global__ void relu_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t n)
{
    pdl_prologue();
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) { T v = x[i]; y[i] = v > T(0) ? v : T(0); }
}
template <typename T> __global__ void relu_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ y, T* __restrict__ dx, int64_t n)
{
    pdl_prologue();
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dx[i] = y[i] > T(0) ? dy[i] : T(0);
}
template <typename T> __global__ void add_kernel(T* __restrict__ acc, const T* __restrict__ o, int64_t n)
{
    pdl_prologue();
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) acc[i] += o[i];
}
// float4 variants for the common aligned float32 case
__global__ void relu_fwd_f4_kernel(const float4* __restrict__ x, float4* __restrict__ y, int64_t n4)
{
    pdl_prologue();
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 v = x[i]; v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f); y[i] = v;
    }
}
__global__ void relu_bwd_f4_kernel(const float4* __restrict__ dy, const float4* __restrict__ y, float4* __restrict__ dx, int64_t n4)
{
    pdl_prologue();
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 g = dy[i], v = y[i];
        g.x = v.x > 0.f ? g.x : 0.f; g.y = v.y > 0.f ? g.y : 0.f; g.z = v.z > 0.f ? g.z : 0.f; g.w = v.w > 0.f ? g.w : 0.f;
        dx[i] = g;
    }
}
__global__ void add_f4_kernel(float4* __restrict__ acc, const float4* __restrict__ o, int64_t n4)
{
    pdl_prologue();
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 a = acc[i], b = o[i]; a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; acc[i] = a;
    }
}
static bool f4_ok(int64_t n, const void* a, const void* b, const void* c)
{
    return (n % 4 == 0) && (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c) % 16 == 0);
}

template <typename T>
__global__ void sgd_kernel(T* __restrict__ w, const T* __restrict__ dw, T* __restrict__ v, int64_t n,
                           T lr, T momentum, T decay, int nesterov)
{
    pdl_prologue();
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        T g = dw[i];
        T vel = momentum * v[i] + g;
        v[i] = vel;
        T wi = w[i];
        if (nesterov) wi -= lr * (decay * wi + g + momentum * vel);
        else wi -= lr * (decay * wi + vel);
        w[i] = wi;
    }
}

// The float32 update four parameters at a time, two float4 groups per trip (the same arithmetic per element).
__global__ void __launch_bounds__(256) sgd_f4_kernel(float4* __restrict__ w, const float4* __restrict__ dw, float4* __restrict__ v, int64_t n4,
                                                     float lr, float momentum, float decay, int nesterov)
{
    pdl_prologue();
    auto one = [&](float g, float& vel, float& wi) {
        vel = momentum * vel + g;
        if (nesterov) wi -= lr * (decay * wi + g + momentum * vel);
        else wi -= lr * (decay * wi + vel);
    };
    auto four = [&](float4 g, float4& ve, float4& wi) { one(g.x, ve.x, wi.x); one(g.y, ve.y, wi.y); one(g.z, ve.z, wi.z); one(g.w, ve.w, wi.w); };
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + stride < n4; i += 2 * stride) {
        const float4 g0 = dw[i], g1 = dw[i + stride];
        float4 v0 = v[i], v1 = v[i + stride], w0 = w[i], w1 = w[i + stride];
        four(g0, v0, w0); four(g1, v1, w1);
        v[i] = v0; w[i] = w0; v[i + stride] = v1; w[i + stride] = w1;
    }
    if (i < n4) {
        const float4 g0 = dw[i];
        float4 v0 = v[i], w0 = w[i];
        four(g0, v0, w0);
        v[i] = v0; w[i] = w0;
    }
}

// ---- pooling -----------------------------------------------------------------------------------

struct PoolP {
    int n, h, w, c, ho, wo, kh, kw, vpad, hpad, vstr, hstr, vdil, hdil;
    int64_t xsn, xsh, xsw, xsc, ysn, ysh, ysw, ysc;
};

// IDX = int when the element count (plus one grid stride) fits 31 bits: the four divisions per element are the
// expensive part of this kernel and 64-bit ones cost several times more.
template <typename T, bool IS_MAX, typename IDX>
__global__ void pool_fwd_kernel(PoolP p, const T* __restrict__ x, T* __restrict__ y, int32_t* __restrict__ idx_max, int nchw)
{
    pdl_prologue();
    const IDX total = (IDX)p.n * p.ho * p.wo * p.c;
    const IDX stride = (IDX)gridDim.x * blockDim.x;
    for (IDX i = (IDX)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        int cc, yy, xx, nn;
        if (nchw) { yy = (int)(i % p.wo); IDX r = i / p.wo; xx = (int)(r % p.ho); r /= p.ho; cc = (int)(r % p.c); nn = (int)(r / p.c); }
        else { cc = (int)(i % p.c); IDX r = i / p.c; yy = (int)(r % p.wo); r /= p.wo; xx = (int)(r % p.ho); nn = (int)(r / p.ho); }
        T best = IS_MAX ? (sizeof(T) == 4 ? (T)(-FLT_MAX) : (T)(-DBL_MAX)) : T(0);
        int bidx = 0, items = 0;
        const T* xb = x + nn * p.xsn + cc * p.xsc;
        for (int ii = 0; ii < p.kh; ii++) {
            int x_x = p.vstr * xx + p.vdil * ii - p.vpad;
            if (x_x < 0 || x_x >= p.h) continue;
            for (int jj = 0; jj < p.kw; jj++) {
                int x_y = p.hstr * yy + p.hdil * jj - p.hpad;
                if (x_y < 0 || x_y >= p.w) continue;
                T v = xb[x_x * p.xsh + x_y * p.xsw];
                if (IS_MAX) { if (v > best) { best = v; bidx = ii * p.kw + jj; } }
                else { best += v; items++; }
            }
        }
        if (IS_MAX) { y[i] = best; if (idx_max) idx_max[i] = bidx; }
        else y[i] = best / (T)items;
    }
}

// NCHW float32 planes that fit shared memory: a block copies a run of whole (image, channel) planes with coalesced
// loads and pools out of shared memory, so the strided, overlapping window reads never reach L2.  Same tap order,
// tie rule (first maximum) and in-bounds divisor as the general kernel: results are bit-identical.
#define B2C_POOL_TILE 8192
template <bool IS_MAX>
__global__ void __launch_bounds__(256) pool_fwd_nchw_planes_kernel(PoolP p, const float* __restrict__ x, float* __restrict__ y,
                                                                   int32_t* __restrict__ idx_max, int planes, int per_block)
{
    pdl_prologue();
    __shared__ float tile[B2C_POOL_TILE];
    const int hw = p.h * p.w, ohw = p.ho * p.wo;
    const int plane0 = blockIdx.x * per_block;
    const int np = planes - plane0 < per_block ? planes - plane0 : per_block;
    const float* src = x + (int64_t)plane0 * hw;
    for (int i = threadIdx.x; i < np * hw; i += 256) tile[i] = src[i];
    __syncthreads();
    for (int o = threadIdx.x; o < np * ohw; o += 256) {
        const int pl = o / ohw, r = o - pl * ohw, xx = r / p.wo, yy = r - xx * p.wo;
        const float* t = tile + pl * hw;
        float best = IS_MAX ? -FLT_MAX : 0.f;
        int bidx = 0, items = 0;
        for (int ii = 0; ii < p.kh; ii++) {
            const int x_x = p.vstr * xx + p.vdil * ii - p.vpad;
            if (x_x < 0 || x_x >= p.h) continue;
            for (int jj = 0; jj < p.kw; jj++) {
                const int x_y = p.hstr * yy + p.hdil * jj - p.hpad;
                if (x_y < 0 || x_y >= p.w) continue;
                const float v = t[x_x * p.w + x_y];
                if (IS_MAX) { if (v > best) { best = v; bidx = ii * p.kw + jj; } }
                else { best += v; items++; }
            }
        }
        const int64_t oi = (int64_t)plane0 * ohw + o;
        if (IS_MAX) { y[oi] = best; if (idx_max) idx_max[oi] = bidx; }
        else y[oi] = best / (float)items;
    }
}

// Backward as a gather over the windows that contain each input element (fixed summation order).
template <typename T, bool IS_MAX>
__global__ void pool_bwd_kernel(PoolP p, const T* __restrict__ dy, const int32_t* __restrict__ idx_max, T* __restrict__ dx, int nchw)
{
    pdl_prologue();
    int64_t total = (int64_t)p.n * p.h * p.w * p.c;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        int cc, iw, ih, nn;
        if (nchw) { iw = (int)(i % p.w); int64_t r = i / p.w; ih = (int)(r % p.h); r /= p.h; cc = (int)(r % p.c); nn = (int)(r / p.c); }
        else { cc = (int)(i % p.c); int64_t r = i / p.c; iw = (int)(r % p.w); r /= p.w; ih = (int)(r % p.h); nn = (int)(r / p.h); }
        T acc = T(0);
        for (int ii = 0; ii < p.kh; ii++) {
            int t = ih + p.vpad - p.vdil * ii;
            if (t < 0 || t % p.vstr) continue;
            int xx = t / p.vstr;
            if (xx >= p.ho) continue;
            for (int jj = 0; jj < p.kw; jj++) {
                int u = iw + p.hpad - p.hdil * jj;
                if (u < 0 || u % p.hstr) continue;
                int yy = u / p.hstr;
                if (yy >= p.wo) continue;
                int64_t o = nn * p.ysn + xx * p.ysh + yy * p.ysw + cc * p.ysc;
                if (IS_MAX) { if (idx_max[o] == ii * p.kw + jj) acc += dy[o]; }
                else {
                    int items = 0;
                    for (int a = 0; a < p.kh; a++) { int q = p.vstr * xx + p.vdil * a - p.vpad; if (q < 0 || q >= p.h) continue;
                        for (int b = 0; b < p.kw; b++) { int r2 = p.hstr * yy + p.hdil * b - p.hpad; if (r2 >= 0 && r2 < p.w) items++; } }
                    acc += dy[o] / (T)items;
                }
            }
        }
        dx[i] = acc;
    }
}


// float32 NHWC pooling with 4 channels per thread (c % 4 == 0).
template <bool IS_MAX>
__global__ void __launch_bounds__(256) pool_fwd_v4_kernel(PoolP p, const float4* __restrict__ x, float4* __restrict__ y, int4* __restrict__ idx_max)
{
    pdl_prologue();
    const int c4 = p.c / 4;
    const int64_t total = (int64_t)p.n * p.ho * p.wo * c4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int cg = (int)(i % c4); int64_t r = i / c4;
        const int yy = (int)(r % p.wo); r /= p.wo;
        const int xx = (int)(r % p.ho); const int nn = (int)(r / p.ho);
        float4 best = IS_MAX ? make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX) : make_float4(0.f, 0.f, 0.f, 0.f);
        int4 bi = make_int4(0, 0, 0, 0);
        int items = 0;
        for (int ii = 0; ii < p.kh; ii++) {
            const int x_x = p.vstr * xx + p.vdil * ii - p.vpad;
            if (x_x < 0 || x_x >= p.h) continue;
            for (int jj = 0; jj < p.kw; jj++) {
                const int x_y = p.hstr * yy + p.hdil * jj - p.hpad;
                if (x_y < 0 || x_y >= p.w) continue;
                const float4 v = x[(((int64_t)nn * p.h + x_x) * p.w + x_y) * c4 + cg];
                if (IS_MAX) {
                    const int t = ii * p.kw + jj;
                    if (v.x > best.x) { best.x = v.x; bi.x = t; }
                    if (v.y > best.y) { best.y = v.y; bi.y = t; }
                    if (v.z > best.z) { best.z = v.z; bi.z = t; }
                    if (v.w > best.w) { best.w = v.w; bi.w = t; }
                } else { best.x += v.x; best.y += v.y; best.z += v.z; best.w += v.w; items++; }
            }
        }
        if (IS_MAX) { y[i] = best; if (idx_max) idx_max[i] = bi; }
        else { const float inv = (float)items; y[i] = make_float4(best.x / inv, best.y / inv, best.z / inv, best.w / inv); }
    }
}

// IDX = int when the element count fits 31 bits: the index decomposition is then done with 32-bit divisions.
template <bool IS_MAX, typename IDX, bool UNIT_DIL>
__global__ void __launch_bounds__(256) pool_bwd_v4_kernel(PoolP p, const float4* __restrict__ dy, const int4* __restrict__ idx_max, float4* __restrict__ dx)
{
    pdl_prologue();
    const int c4 = p.c / 4;
    const IDX total = (IDX)p.n * p.h * p.w * c4;
    for (IDX i = (IDX)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (IDX)gridDim.x * blockDim.x) {
        const int cg = (int)(i % c4); IDX r = i / c4;
        const int iw = (int)(r % p.w); r /= p.w;
        const int ih = (int)(r % p.h); const int nn = (int)(r / p.h);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        // Windows that contain this element, in ascending tap order.  With dilation 1 (UNIT_DIL) the taps that can reach
        // it are ii0, ii0 + vstr, ... with ii0 = (ih + vpad) mod vstr, and the window row falls by one per step: one
        // division per axis instead of a modulo and a division per tap.
        const int th = ih + p.vpad, tw = iw + p.hpad;
        const int ii0 = UNIT_DIL ? th % p.vstr : 0, ii_step = UNIT_DIL ? p.vstr : 1, xx0 = UNIT_DIL ? th / p.vstr : 0;
        const int jj0 = UNIT_DIL ? tw % p.hstr : 0, jj_step = UNIT_DIL ? p.hstr : 1, yy0 = UNIT_DIL ? tw / p.hstr : 0;
        for (int ii = ii0, ka = 0; ii < p.kh; ii += ii_step, ka++) {
            int xx;
            if (UNIT_DIL) { xx = xx0 - ka; if (xx < 0) break; }
            else { const int t = th - p.vdil * ii; if (t < 0 || t % p.vstr) continue; xx = t / p.vstr; }
            if (xx >= p.ho) continue;
            for (int jj = jj0, kb = 0; jj < p.kw; jj += jj_step, kb++) {
                int yy;
                if (UNIT_DIL) { yy = yy0 - kb; if (yy < 0) break; }
                else { const int u = tw - p.hdil * jj; if (u < 0 || u % p.hstr) continue; yy = u / p.hstr; }
                if (yy >= p.wo) continue;
                const int64_t o = (((int64_t)nn * p.ho + xx) * p.wo + yy) * c4 + cg;
                const float4 g = dy[o];
                if (IS_MAX) {
                    const int4 id = idx_max[o];
                    const int tap = ii * p.kw + jj;
                    if (id.x == tap) acc.x += g.x;
                    if (id.y == tap) acc.y += g.y;
                    if (id.z == tap) acc.z += g.z;
                    if (id.w == tap) acc.w += g.w;
                } else {
                    int items = 0;
                    for (int a = 0; a < p.kh; a++) { int q = p.vstr * xx + p.vdil * a - p.vpad; if (q < 0 || q >= p.h) continue;
                        for (int b = 0; b < p.kw; b++) { int r2 = p.hstr * yy + p.hdil * b - p.hpad; if (r2 >= 0 && r2 < p.w) items++; } }
                    const float inv = (float)items;
                    acc.x += g.x / inv; acc.y += g.y / inv; acc.z += g.z / inv; acc.w += g.w / inv;
                }
            }
        }
        dx[i] = acc;
    }
}

// Max pooling backward for the 3x3 window with stride 2 and dilation 1 (the pool after a network's stem), NHWC float4:
// the same gather as pool_bwd_v4_kernel with the window arithmetic in constants.  An element (ih, iw) is reached by
// tap ii = (ih + vpad) % 2 (and ii + 2 when that is 0) of window row (ih + vpad) / 2 (and the row before it); the same
// along w.  Grid (blocks over iw x channel groups, n x h): one division per thread.  Taps are visited in ascending
// order, as the general kernel does, so the sums are the same bits.
__global__ void __launch_bounds__(256) pool_bwd_max_k3s2_kernel(PoolP p, const float4* __restrict__ dy, const int4* __restrict__ idx_max,
                                                                float4* __restrict__ dx)
{
    pdl_prologue();
    const int c4 = p.c / 4;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= p.w * c4) return;
    const int iw = e / c4, cg = e - iw * c4;
    const int nn = blockIdx.y / p.h, ih = blockIdx.y - nn * p.h;
    const int th = ih + p.vpad, tw = iw + p.hpad;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int ka = 0; ka < 2; ka++) {
        const int ii = (th & 1) + 2 * ka, xx = (th >> 1) - ka;
        if (ii > 2 || xx < 0 || xx >= p.ho) continue;
#pragma unroll
        for (int kb = 0; kb < 2; kb++) {
            const int jj = (tw & 1) + 2 * kb, yy = (tw >> 1) - kb;
            if (jj > 2 || yy < 0 || yy >= p.wo) continue;
            const int64_t o = (((int64_t)nn * p.ho + xx) * p.wo + yy) * c4 + cg;
            const float4 g = dy[o];
            const int4 id = idx_max[o];
            const int tap = ii * 3 + jj;
            if (id.x == tap) acc.x += g.x;
            if (id.y == tap) acc.y += g.y;
            if (id.z == tap) acc.z += g.z;
            if (id.w == tap) acc.w += g.w;
        }
    }
    dx[((int64_t)blockIdx.y * p.w + iw) * c4 + cg] = acc;
}

// out = max(a + b, 0)  (residual sum followed by ReLU in one pass)
__global__ void add_relu_f4_kernel(const float4* __restrict__ a, const float4* __restrict__ b, float4* __restrict__ out, int64_t n4)
{
    pdl_prologue();
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 u = a[i], v = b[i];
        out[i] = make_float4(fmaxf(u.x + v.x, 0.f), fmaxf(u.y + v.y, 0.f), fmaxf(u.z + v.z, 0.f), fmaxf(u.w + v.w, 0.f));
    }
}
template <typename T> __global__ void add_relu_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, int64_t n)
{
    pdl_prologue();
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) { T v = a[i] + b[i]; out[i] = v > T(0) ? v : T(0); }
}

// dx = (y > 0) ? a + b : 0  (the input-gradient sum of an addition block and the backward of the ReLU before it)
__global__ void add_relu_bwd_f4_kernel(const float4* __restrict__ a, const float4* __restrict__ b, const float4* __restrict__ y,
                                       float4* __restrict__ dx, int64_t n4)
{
    pdl_prologue();
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 u = a[i], v = b[i], m = y[i];
        dx[i] = make_float4(m.x > 0.f ? __fadd_rn(u.x, v.x) : 0.f, m.y > 0.f ? __fadd_rn(u.y, v.y) : 0.f,
                            m.z > 0.f ? __fadd_rn(u.z, v.z) : 0.f, m.w > 0.f ? __fadd_rn(u.w, v.w) : 0.f);
    }
}
template <typename T> __global__ void add_relu_bwd_kernel(const T* __restrict__ a, const T* __restrict__ b, const T* __restrict__ y,
                                                          T* __restrict__ dx, int64_t n)
{
    pdl_prologue();
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dx[i] = y[i] > T(0) ? a[i] + b[i] : T(0);
}

// ---- softmax / cross-entropy -------------------------------------------------------------------

template <typename T> __device__ T block_reduce(T v, T* sm, bool is_max)
{
    int t = threadIdx.x;
    sm[t] = v; __syncthreads();
    for (int s = blockDim.x / 2; s > 0; s >>= 1) {
        if (t < s) sm[t] = is_max ? (sm[t] > sm[t + s] ? sm[t] : sm[t + s]) : (sm[t] + sm[t + s]);
        __syncthreads();
    }
    T r = sm[0]; __syncthreads();
    return r;
}

template <typename T>
__global__ void softmax_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int cols)
{
    pdl_prologue();
    __shared__ T sm[256];
    const T* xr = x + (int64_t)blockIdx.x * cols; T* yr = y + (int64_t)blockIdx.x * cols;
    T mx = sizeof(T) == 4 ? (T)(-FLT_MAX) : (T)(-DBL_MAX);
    for (int j = threadIdx.x; j < cols; j += blockDim.x) mx = xr[j] > mx ? xr[j] : mx;
    mx = block_reduce<T>(mx, sm, true);
    T s = T(0);
    for (int j = threadIdx.x; j < cols; j += blockDim.x) { T e = exp(xr[j] - mx); yr[j] = e; s += e; }
    s = block_reduce<T>(s, sm, false);
    for (int j = threadIdx.x; j < cols; j += blockDim.x) yr[j] = yr[j] / s;
}

template <typename T>
__global__ void softmax_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ y, T* __restrict__ dx, int cols)
{
    pdl_prologue();
    __shared__ T sm[256];
    const T* dr = dy + (int64_t)blockIdx.x * cols; const T* yr = y + (int64_t)blockIdx.x * cols; T* xr = dx + (int64_t)blockIdx.x * cols;
    T s = T(0);
    for (int j = threadIdx.x; j < cols; j += blockDim.x) s += dr[j] * yr[j];
    s = block_reduce<T>(s, sm, false);
    for (int j = threadIdx.x; j < cols; j += blockDim.x) xr[j] = yr[j] * (dr[j] - s);
}

template <typename T>
__global__ void cce_kernel(const T* __restrict__ probs, const int32_t* __restrict__ labels, int cols, int global_batch,
                           T eps, T* __restrict__ row_loss, int32_t* __restrict__ hit, T* __restrict__ dx)
{
    pdl_prologue();
    __shared__ T smv[256]; __shared__ int smi[256];
    const T* pr = probs + (int64_t)blockIdx.x * cols; T* xr = dx + (int64_t)blockIdx.x * cols;
    int label = labels[blockIdx.x];
    T best = sizeof(T) == 4 ? (T)(-FLT_MAX) : (T)(-DBL_MAX); int bi = 0x7fffffff;
    for (int j = threadIdx.x; j < cols; j += blockDim.x) {
        T v = pr[j];
        if (v > best) { best = v; bi = j; }
        xr[j] = T(0);
    }
    smv[threadIdx.x] = best; smi[threadIdx.x] = bi; __syncthreads();
    for (int s = blockDim.x / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) {
            T ov = smv[threadIdx.x + s]; int oi = smi[threadIdx.x + s];
            if (ov > smv[threadIdx.x] || (ov == smv[threadIdx.x] && oi < smi[threadIdx.x])) { smv[threadIdx.x] = ov; smi[threadIdx.x] = oi; }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        bool in_range = label >= 0 && label < cols;
        T pred = in_range ? pr[label] : eps;
        if (pred < eps) pred = eps; else if (pred > (T(1) - eps)) pred = T(1) - eps;
        row_loss[blockIdx.x] = log(pred);
        if (hit) hit[blockIdx.x] = (in_range && smi[0] == label) ? 1 : 0;
    }
    __syncthreads();
    if (threadIdx.x == 0 && label >= 0 && label < cols) {
        T pred = pr[label];
        if (pred < eps) pred = eps; else if (pred > (T(1) - eps)) pred = T(1) - eps;
        xr[label] = T(1) / (-pred * (T)global_batch);
    }
}

// Totals of the loss kernel's per-row outputs: out[0] = -sum(row_loss) / rows (the mean loss), out[1] = 100 * hits /
// rows (accuracy in per cent).  One block; every thread adds its rows in index order in double, then a fixed tree.
template <typename T>
__global__ void cce_totals_kernel(const T* __restrict__ row_loss, const int32_t* __restrict__ hit, int rows, double* __restrict__ out)
{
    pdl_prologue();
    __shared__ double s0[256], s1[256];
    double a0 = 0.0, a1 = 0.0;
    for (int i = threadIdx.x; i < rows; i += 256) { a0 += (double)row_loss[i]; a1 += hit ? (double)hit[i] : 0.0; }
    s0[threadIdx.x] = a0; s1[threadIdx.x] = a1;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if (threadIdx.x < s) { s0[threadIdx.x] += s0[threadIdx.x + s]; s1[threadIdx.x] += s1[threadIdx.x + s]; }
        __syncthreads();
    }
    if (threadIdx.x == 0) { out[0] = -s0[0] / (double)rows; out[1] = 100.0 * s1[0] / (double)rows; }
}

// inv_std[c] = 1 / sqrt(var[c] + eps), evaluated in double and rounded once (what NumPy gives for a float64
// intermediate): the per-channel factor of the inference-mode batch norm.
template <typename T>
__global__ void bn_inv_std_kernel(const T* __restrict__ var, int c, double eps, T* __restrict__ inv_std)
{
    pdl_prologue();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < c) inv_std[i] = (T)(1.0 / sqrt((double)var[i] + eps));
}

// Register-resident chains of dependent fused multiply-adds: 8 independent chains per thread, `iters` rounds.
// Measures the FMA issue rate of the device for the roofline denominator of the FMA engine (no memory traffic).
template <typename T>
__global__ void __launch_bounds__(256) fma_probe_kernel(int iters, T seed, T* __restrict__ sink)
{
    pdl_prologue();
    T a[8];
#pragma unroll
    for (int k = 0; k < 8; k++) a[k] = seed + (T)(threadIdx.x + k);
    const T m = (T)0.999, b = (T)1e-3;
    for (int i = 0; i < iters; i++) {
#pragma unroll
        for (int k = 0; k < 8; k++) a[k] = a[k] * m + b;
    }
    T s = a[0];
#pragma unroll
    for (int k = 1; k < 8; k++) s += a[k];
    if (s == (T)-1) sink[blockIdx.x * blockDim.x + threadIdx.x] = s;     // never true: keeps the chains alive
}

}  // namespace b2c

// ================================= C ABI ==========================================================
using namespace b2c;

#define CHECK_DTYPE(d) do { if ((d) != B2C_F32 && (d) != B2C_F64) return B2C_ERR_BAD_ENUM; } while (0)
#define CHECK_LAYOUT(l) do { if ((l) != B2C_LAYOUT_NHWC && (l) != B2C_LAYOUT_NCHW) return B2C_ERR_BAD_ENUM; } while (0)

extern "C" int b2c_bn_train_forward(int dtype, int layout, int n, int c, int hw, const void* x, const void* gamma,
                                    const void* beta, void* running_mean, void* running_var, double momentum,
                                    double eps, int fuse_relu, void* y, void* save_mean, void* save_inv_std,
                                    void* scratch, size_t scratch_bytes, void* stream)
{
    CHECK_DTYPE(dtype); CHECK_LAYOUT(layout);
    if (!x || !gamma || !beta || !running_mean || !running_var || !y || !save_mean || !save_inv_std || !scratch) return B2C_ERR_NULL_POINTER;
    if (n <= 0 || c <= 0 || hw <= 0) return B2C_ERR_BAD_GEOMETRY;
    if (scratch_bytes < reduce2_bytes(c)) return B2C_ERR_WORKSPACE_TOO_SMALL;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == B2C_F32)
        return bn_train_forward_t<float>(layout, n, c, hw, (const float*)x, (const float*)gamma, (const float*)beta, (float*)running_mean,
                                         (float*)running_var, momentum, eps, fuse_relu, (float*)y, (float*)save_mean, (float*)save_inv_std, (double*)scratch, scratch_bytes, st);
    return bn_train_forward_t<double>(layout, n, c, hw, (const double*)x, (const double*)gamma, (const double*)beta, (double*)running_mean,
                                      (double*)running_var, momentum, eps, fuse_relu, (double*)y, (double*)save_mean, (double*)save_inv_std, (double*)scratch, scratch_bytes, st);
}

extern "C" int b2c_bn_train_forward_residual(int dtype, int layout, int n, int c, int hw, const void* x, const void* gamma,
                                             const void* beta, void* running_mean, void* running_var, double momentum,
                                             double eps, const void* addend, int relu, void* y, void* save_mean,
                                             void* save_inv_std, void* scratch, size_t scratch_bytes, void* stream)
{
    CHECK_DTYPE(dtype); CHECK_LAYOUT(layout);
    if (!x || !gamma || !beta || !running_mean || !running_var || !addend || !y || !save_mean || !save_inv_std || !scratch) return B2C_ERR_NULL_POINTER;
    if (n <= 0 || c <= 0 || hw <= 0) return B2C_ERR_BAD_GEOMETRY;
    if (scratch_bytes < reduce2_bytes(c)) return B2C_ERR_WORKSPACE_TOO_SMALL;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == B2C_F32)
        return bn_train_forward_t<float>(layout, n, c, hw, (const float*)x, (const float*)gamma, (const float*)beta, (float*)running_mean,
                                         (float*)running_var, momentum, eps, relu, (float*)y, (float*)save_mean, (float*)save_inv_std,
                                         (double*)scratch, scratch_bytes, st, (const float*)addend);
    return bn_train_forward_t<double>(layout, n, c, hw, (const double*)x, (const double*)gamma, (const double*)beta, (double*)running_mean,
                                      (double*)running_var, momentum, eps, relu, (double*)y, (double*)save_mean, (double*)save_inv_std,
                                      (double*)scratch, scratch_bytes, st, (const double*)addend);
}

// ---- batch-norm forward without caller-supplied scratch ----------------------------------------
// Some hosts of this library hand all device memory to their own pool when they start and from then
// on refuse to allocate: a late cudaMalloc synchronises the whole device, can fragment or simply fail
// once the pool owns the card, and a training or serving loop with a latency budget cannot absorb
// that.  Such a caller may have no spare buffer to lend as reduction scratch either.  For them the
// per-channel partial sums of this one kernel live in a fixed array inside the library image
// (2 MiB per GPU that loads the library, held until the process exits).
#define B2C_STATIC_SCRATCH_DOUBLES (64 * 2 * 2048)      // 64 row chunks x (sum, sum of squares) x 2048 channels
#define B2C_STATIC_MAX_CHANNELS 2048
static __device__ __align__(256) double g_bn_static_scratch[B2C_STATIC_SCRATCH_DOUBLES];

// In host code the array's name is only a handle for the runtime, not a device address; the address
// the kernels need is looked up once per device (with that device current) and kept.
static double* g_bn_static_ptr[64] = {nullptr};
static std::mutex g_bn_static_mutex;

static int bn_static_scratch(double** out)
{
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { b2c::set_cuda_error(e, "cudaGetDevice"); return B2C_ERR_CUDA; }
    if (dev < 0 || dev >= 64) return B2C_ERR_TOO_LARGE;
    std::lock_guard<std::mutex> lock(g_bn_static_mutex);
    if (!g_bn_static_ptr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_bn_static_scratch);
        if (e != cudaSuccess || !p) { b2c::set_cuda_error(e, "cudaGetSymbolAddress(g_bn_static_scratch)"); return B2C_ERR_CUDA; }
        g_bn_static_ptr[dev] = (double*)p;
    }
    *out = g_bn_static_ptr[dev];
    return B2C_OK;
}

extern "C" int b2c_bn_train_forward_static(int dtype, int layout, int n, int c, int hw, const void* x, const void* gamma,
                                           const void* beta, void* running_mean, void* running_var, double momentum,
                                           double eps, int fuse_relu, void* y, void* save_mean, void* save_inv_std,
                                           void* stream)
{
    CHECK_DTYPE(dtype); CHECK_LAYOUT(layout);
    if (!x || !gamma || !beta || !running_mean || !running_var || !y || !save_mean || !save_inv_std) return B2C_ERR_NULL_POINTER;
    if (n <= 0 || c <= 0 || hw <= 0) return B2C_ERR_BAD_GEOMETRY;
    if (c > B2C_STATIC_MAX_CHANNELS) return B2C_ERR_TOO_LARGE;     // the fixed array holds 64 chunks of at most 2048 channels
    double* scratch = nullptr;
    int rc = bn_static_scratch(&scratch);
    if (rc) return rc;
    const size_t scratch_bytes = sizeof(double) * B2C_STATIC_SCRATCH_DOUBLES;
    cudaStream_t st = (cudaStream_t)stream;
    // Every partial the second stage reads is written by the first stage of the same call, so the
    // previous call's contents never need clearing.
    if (dtype == B2C_F32)
        return bn_train_forward_t<float>(layout, n, c, hw, (const float*)x, (const float*)gamma, (const float*)beta, (float*)running_mean,
                                         (float*)running_var, momentum, eps, fuse_relu, (float*)y, (float*)save_mean, (float*)save_inv_std,
                                         scratch, scratch_bytes, st);
    return bn_train_forward_t<double>(layout, n, c, hw, (const double*)x, (const double*)gamma, (const double*)beta, (double*)running_mean,
                                      (double*)running_var, momentum, eps, fuse_relu, (double*)y, (double*)save_mean, (double*)save_inv_std,
                                      scratch, scratch_bytes, st);
}

extern "C" int b2c_bn_train_forward_prestats(int n, int c, int hw, const void* x, const void* stats, size_t stats_bytes,
                                             const void* gamma, const void* beta, void* running_mean, void* running_var,
                                             double momentum, double eps, int fuse_relu, const void* addend, void* y,
                                             void* save_mean, void* save_inv_std, void* scratch, size_t scratch_bytes, void* stream)
{
    if (!x || !stats || !gamma || !beta || !running_mean || !running_var || !y || !save_mean || !save_inv_std || !scratch) return B2C_ERR_NULL_POINTER;
    if (n <= 0 || c <= 0 || hw <= 0) return B2C_ERR_BAD_GEOMETRY;
    if (!v4_ok(B2C_F32, B2C_LAYOUT_NHWC, c, x, y, addend ? addend : x)) return B2C_ERR_UNSUPPORTED;
    // the convolution chose how many rows of sums to leave (one per 32 output rows, or one per CTA group and row
    // quadrant): the byte count it reported for the buffer says which
    const size_t row_bytes = (size_t)2 * c * sizeof(float);
    if (stats_bytes < row_bytes || stats_bytes % row_bytes || stats_bytes / row_bytes > (size_t)(((int64_t)n * hw + 127) / 128) * 4)
        return B2C_ERR_BAD_GEOMETRY;
    if (scratch_bytes < reduce2_bytes(c)) return B2C_ERR_WORKSPACE_TOO_SMALL;
    const int rows = (int)(stats_bytes / row_bytes);
    cudaStream_t st = (cudaStream_t)stream;
    if (rows <= 1024) {
        // few rows: one kernel adds them and finishes the statistics
        launch_pdl(bn_rows_final_kernel, (c + 31) / 32, dim3(32, 32), 0, st, (const float*)stats, rows, c, (double)n * hw, momentum, eps,
                   (float*)save_mean, (float*)save_inv_std, (float*)running_mean, (float*)running_var);
        int rc = check_launch("bn_rows_final"); if (rc) return rc;
        V4Geo ga = v4_apply_geo((int64_t)n * hw, c);
        launch_pdl(bn_apply_v4_kernel, dim3(ga.gx, ga.chunks), 256, 0, st, (const float4*)x, (float4*)y, (const float*)save_mean, (const float*)save_inv_std,
                                                                  (const float*)gamma, (const float*)beta, ga, fuse_relu, (const float4*)addend);
        return check_launch("bn_apply_v4");
    }
    // chunks: at least 32 rows of sums each, about two blocks per SM, no more than the scratch holds
    const int gx = (c + 31) / 32;
    int chunks = (296 + gx - 1) / gx;
    if (chunks > rows / 32) chunks = rows / 32;
    const int max_chunks = (int)(scratch_bytes / ((size_t)2 * c * sizeof(double)));
    if (chunks > max_chunks) chunks = max_chunks;
    if (chunks < 1) chunks = 1;
    launch_pdl(bn_conv_sums_kernel, dim3(gx, chunks), dim3(32, 8), 0, st, (const float*)stats, rows, c, (double*)scratch);
    int rc = check_launch("bn_conv_sums"); if (rc) return rc;
    rc = final_warp((const double*)scratch, chunks, c, 0, (double)n * hw, momentum, eps, (float*)save_mean, (float*)save_inv_std,
                    (float*)running_mean, (float*)running_var, st);
    if (rc) return rc;
    V4Geo ga = v4_apply_geo((int64_t)n * hw, c);
    launch_pdl(bn_apply_v4_kernel, dim3(ga.gx, ga.chunks), 256, 0, st, (const float4*)x, (float4*)y, (const float*)save_mean, (const float*)save_inv_std,
                                                              (const float*)gamma, (const float*)beta, ga, fuse_relu, (const float4*)addend);
    return check_launch("bn_apply_v4");
}

extern "C" int b2c_bn_train_backward(int dtype, int layout, int n, int c, int hw, const void* x, const void* dy,
                                     const void* y_for_relu_mask, const void* beta_for_relu_mask, const void* gamma, const void* save_mean,
                                     const void* save_inv_std, void* dgamma, void* dbeta, void* dx,
                                     void* scratch, size_t scratch_bytes, void* stream)
{
    CHECK_DTYPE(dtype); CHECK_LAYOUT(layout);
    if (!x || !dy || !gamma || !save_mean || !save_inv_std || !dgamma || !dbeta || !scratch) return B2C_ERR_NULL_POINTER;
    if (n <= 0 || c <= 0 || hw <= 0) return B2C_ERR_BAD_GEOMETRY;
    if (scratch_bytes < reduce2_bytes(c)) return B2C_ERR_WORKSPACE_TOO_SMALL;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == B2C_F32)
        return bn_train_backward_t<float>(layout, n, c, hw, (const float*)x, (const float*)dy, (const float*)y_for_relu_mask,
                                          (const float*)beta_for_relu_mask, (const float*)gamma,
                                          (const float*)save_mean, (const float*)save_inv_std, (float*)dgamma, (float*)dbeta, (float*)dx, (double*)scratch, scratch_bytes, st);
    return bn_train_backward_t<double>(layout, n, c, hw, (const double*)x, (const double*)dy, (const double*)y_for_relu_mask,
                                       (const double*)beta_for_relu_mask, (const double*)gamma,
                                       (const double*)save_mean, (const double*)save_inv_std, (double*)dgamma, (double*)dbeta, (double*)dx, (double*)scratch, scratch_bytes, st);
}

extern "C" int b2c_bn_inference(int dtype, int layout, int n, int c, int hw, const void* x, const void* mean,
                                const void* inv_std, const void* gamma, const void* beta, int relu, void* y, void* stream)
{
    CHECK_DTYPE(dtype); CHECK_LAYOUT(layout);
    if (!x || !mean || !inv_std || !gamma || !beta || !y) return B2C_ERR_NULL_POINTER;
    if (n <= 0 || c <= 0 || hw <= 0) return B2C_ERR_BAD_GEOMETRY;
    cudaStream_t st = (cudaStream_t)stream;
    int64_t total = (int64_t)n * c * hw;
    if (v4_ok(dtype, layout, c, x, y, x)) {
        V4Geo ga = v4_apply_geo((int64_t)n * hw, c);
        launch_pdl(bn_apply_v4_kernel, dim3(ga.gx, ga.chunks), 256, 0, st, (const float4*)x, (float4*)y, (const float*)mean, (const float*)inv_std,
                                                                  (const float*)gamma, (const float*)beta, ga, relu, (const float4*)nullptr);
        return check_launch("bn_inference_v4");
    }
    if (dtype == B2C_F32)
        launch_pdl(bn_apply_kernel<float>, ew_blocks(total), 256, 0, st, (const float*)x, (float*)y, (const float*)mean, (const float*)inv_std,
                                                                (const float*)gamma, (const float*)beta, total, c, hw, layout == B2C_LAYOUT_NCHW, relu, 1, (const float*)nullptr);
    else
        launch_pdl(bn_apply_kernel<double>, ew_blocks(total), 256, 0, st, (const double*)x, (double*)y, (const double*)mean, (const double*)inv_std,
                                                                 (const double*)gamma, (const double*)beta, total, c, hw, layout == B2C_LAYOUT_NCHW, relu, 1, (const double*)nullptr);
    return check_launch("bn_inference");
}

extern "C" int b2c_relu_forward(int dtype, int64_t count, const void* x, void* y, void* stream)
{
    CHECK_DTYPE(dtype);
    if (!x || !y) return B2C_ERR_NULL_POINTER;
    if (count < 0) return B2C_ERR_BAD_GEOMETRY;
    if (count == 0) return B2C_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == B2C_F32) {
        if (f4_ok(count, x, y, y)) launch_pdl(relu_fwd_f4_kernel, ew_blocks(count / 4), 256, 0, st, (const float4*)x, (float4*)y, count / 4);
        else launch_pdl(relu_fwd_kernel<float>, ew_blocks(count), 256, 0, st, (const float*)x, (float*)y, count);
    } else launch_pdl(relu_fwd_kernel<double>, ew_blocks(count), 256, 0, st, (const double*)x, (double*)y, count);
    return check_launch("relu_forward");
}

extern "C" int b2c_relu_backward(int dtype, int64_t count, const void* dy, const void* y, void* dx, void* stream)
{
    CHECK_DTYPE(dtype);
    if (!dy || !y || !dx) return B2C_ERR_NULL_POINTER;
    if (count < 0) return B2C_ERR_BAD_GEOMETRY;
    if (count == 0) return B2C_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == B2C_F32) {
        if (f4_ok(count, dy, y, dx)) launch_pdl(relu_bwd_f4_kernel, ew_blocks(count / 4), 256, 0, st, (const float4*)dy, (const float4*)y, (float4*)dx, count / 4);
        else launch_pdl(relu_bwd_kernel<float>, ew_blocks(count), 256, 0, st, (const float*)dy, (const float*)y, (float*)dx, count);
    } else launch_pdl(relu_bwd_kernel<double>, ew_blocks(count), 256, 0, st, (const double*)dy, (const double*)y, (double*)dx, count);
    return check_launch("relu_backward");
}

extern "C" int b2c_add_inplace(int dtype, int64_t count, void* acc, const void* other, void* stream)
{
    CHECK_DTYPE(dtype);
    if (!acc || !other) return B2C_ERR_NULL_POINTER;
    if (count < 0) return B2C_ERR_BAD_GEOMETRY;
    if (count == 0) return B2C_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == B2C_F32) {
        if (f4_ok(count, acc, other, acc)) launch_pdl(add_f4_kernel, ew_blocks(count / 4), 256, 0, st, (float4*)acc, (const float4*)other, count / 4);
        else launch_pdl(add_kernel<float>, ew_blocks(count), 256, 0, st, (float*)acc, (const float*)other, count);
    } else launch_pdl(add_kernel<double>, ew_blocks(count), 256, 0, st, (double*)acc, (const double*)other, count);
    return check_launch("add_inplace");
}

extern "C" int b2c_add_relu(int dtype, int64_t count, const void* a, const void* b, void* out, void* stream)
{
    CHECK_DTYPE(dtype);
    if (!a || !b || !out) return B2C_ERR_NULL_POINTER;
    if (count < 0) return B2C_ERR_BAD_GEOMETRY;
    if (count == 0) return B2C_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == B2C_F32) {
        if (f4_ok(count, a, b, out)) launch_pdl(add_relu_f4_kernel, ew_blocks(count / 4), 256, 0, st, (const float4*)a, (const float4*)b, (float4*)out, count / 4);
        else launch_pdl(add_relu_kernel<float>, ew_blocks(count), 256, 0, st, (const float*)a, (const float*)b, (float*)out, count);
    } else launch_pdl(add_relu_kernel<double>, ew_blocks(count), 256, 0, st, (const double*)a, (const double*)b, (double*)out, count);
    return check_launch("add_relu");
}

extern "C" int b2c_add_relu_backward(int dtype, int64_t count, const void* a, const void* b, const void* y, void* dx, void* stream)
{
    CHECK_DTYPE(dtype);
    if (!a || !b || !y || !dx) return B2C_ERR_NULL_POINTER;
    if (count < 0) return B2C_ERR_BAD_GEOMETRY;
    if (count == 0) return B2C_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == B2C_F32) {
        if (f4_ok(count, a, b, dx) && ((uintptr_t)y & 15) == 0)
            launch_pdl(add_relu_bwd_f4_kernel, ew_blocks(count / 4), 256, 0, st, (const float4*)a, (const float4*)b, (const float4*)y, (float4*)dx, count / 4);
        else launch_pdl(add_relu_bwd_kernel<float>, ew_blocks(count), 256, 0, st, (const float*)a, (const float*)b, (const float*)y, (float*)dx, count);
    } else launch_pdl(add_relu_bwd_kernel<double>, ew_blocks(count), 256, 0, st, (const double*)a, (const double*)b, (const double*)y, (double*)dx, count);
    return check_launch("add_relu_backward");
}

static int make_pool(PoolP& p, int layout, int n, int h, int w, int c, int kh, int kw, int vpad, int hpad, int vstr,
                     int hstr, int vdil, int hdil)
{
    if (n <= 0 || h <= 0 || w <= 0 || c <= 0 || kh <= 0 || kw <= 0 || vpad < 0 || hpad < 0 || vstr < 1 || hstr < 1 || vdil < 1 || hdil < 1)
        return B2C_ERR_BAD_GEOMETRY;
    int eh = h + 2 * vpad - vdil * (kh - 1) - 1, ew = w + 2 * hpad - hdil * (kw - 1) - 1;
    if (eh < 0 || ew < 0) return B2C_ERR_BAD_GEOMETRY;
    p.n = n; p.h = h; p.w = w; p.c = c; p.kh = kh; p.kw = kw; p.vpad = vpad; p.hpad = hpad; p.vstr = vstr; p.hstr = hstr; p.vdil = vdil; p.hdil = hdil;
    p.ho = eh / vstr + 1; p.wo = ew / hstr + 1;
    ActStride xs = act_stride(layout, h, w, c), ys = act_stride(layout, p.ho, p.wo, c);
    p.xsn = xs.sn; p.xsh = xs.sh; p.xsw = xs.sw; p.xsc = xs.sc; p.ysn = ys.sn; p.ysh = ys.sh; p.ysw = ys.sw; p.ysc = ys.sc;
    return B2C_OK;
}

extern "C" int b2c_pool_forward(int dtype, int layout, int is_max, int n, int h, int w, int c, int kh, int kw,
                                int vpad, int hpad, int vstr, int hstr, int vdil, int hdil,
                                const void* x, void* y, int32_t* idx_max, void* stream)
{
    CHECK_DTYPE(dtype); CHECK_LAYOUT(layout);
    if (!x || !y) return B2C_ERR_NULL_POINTER;
    PoolP p; int rc = make_pool(p, layout, n, h, w, c, kh, kw, vpad, hpad, vstr, hstr, vdil, hdil); if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    int64_t total = (int64_t)n * p.ho * p.wo * c; int nchw = layout == B2C_LAYOUT_NCHW;
    if (dtype == B2C_F32 && !nchw && c % 4 == 0 && (((uintptr_t)x | (uintptr_t)y | (uintptr_t)idx_max) & 15) == 0) {
        if (is_max) launch_pdl(pool_fwd_v4_kernel<true>, ew_blocks(total / 4), 256, 0, st, p, (const float4*)x, (float4*)y, (int4*)idx_max);
        else launch_pdl(pool_fwd_v4_kernel<false>, ew_blocks(total / 4), 256, 0, st, p, (const float4*)x, (float4*)y, (int4*)idx_max);
        return check_launch("pool_forward_v4");
    }
    if (dtype == B2C_F32 && nchw && (int64_t)h * w <= B2C_POOL_TILE && (int64_t)n * c < 0x7fffffffLL) {
        const int planes = n * c;
        int per_block = B2C_POOL_TILE / (h * w);
        if (per_block > 16) per_block = 16;
        const int blocks = (planes + per_block - 1) / per_block;
        if (is_max) launch_pdl(pool_fwd_nchw_planes_kernel<true>, blocks, 256, 0, st, p, (const float*)x, (float*)y, idx_max, planes, per_block);
        else launch_pdl(pool_fwd_nchw_planes_kernel<false>, blocks, 256, 0, st, p, (const float*)x, (float*)y, idx_max, planes, per_block);
        return check_launch("pool_forward_nchw_planes");
    }
    // 32-bit index arithmetic when the output count, one grid stride and the input offsets all fit
    const bool small = total + (int64_t)ew_blocks(total) * 256 < 0x7fffffffLL && (int64_t)n * h * w * c < 0x7fffffffLL;
#define B2C_POOL_FWD(T, MAXF)                                                                                              \
    do {                                                                                                                   \
        if (small) launch_pdl(pool_fwd_kernel<T, MAXF, int>, ew_blocks(total), 256, 0, st, p, (const T*)x, (T*)y, idx_max, nchw); \
        else launch_pdl(pool_fwd_kernel<T, MAXF, int64_t>, ew_blocks(total), 256, 0, st, p, (const T*)x, (T*)y, idx_max, nchw);   \
    } while (0)
    if (dtype == B2C_F32) { if (is_max) B2C_POOL_FWD(float, true); else B2C_POOL_FWD(float, false); }
    else { if (is_max) B2C_POOL_FWD(double, true); else B2C_POOL_FWD(double, false); }
#undef B2C_POOL_FWD
    return check_launch("pool_forward");
}

extern "C" int b2c_pool_backward(int dtype, int layout, int is_max, int n, int h, int w, int c, int kh, int kw,
                                 int vpad, int hpad, int vstr, int hstr, int vdil, int hdil,
                                 const void* dy, const int32_t* idx_max, void* dx, void* stream)
{
    CHECK_DTYPE(dtype); CHECK_LAYOUT(layout);
    if (!dy || !dx || (is_max && !idx_max)) return B2C_ERR_NULL_POINTER;
    PoolP p; int rc = make_pool(p, layout, n, h, w, c, kh, kw, vpad, hpad, vstr, hstr, vdil, hdil); if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    int64_t total = (int64_t)n * h * w * c; int nchw = layout == B2C_LAYOUT_NCHW;
    if (dtype == B2C_F32 && !nchw && c % 4 == 0 && (((uintptr_t)dy | (uintptr_t)dx | (uintptr_t)idx_max) & 15) == 0) {
        const bool small = total / 4 + (int64_t)ew_blocks(total / 4) * 256 < 0x7fffffffLL;
        const bool unit = vdil == 1 && hdil == 1;
#define B2C_POOL_BWD_V4(MAXF, IDXT)                                                                                                         \
        do {                                                                                                                                \
            if (unit) launch_pdl(pool_bwd_v4_kernel<MAXF, IDXT, true>, ew_blocks(total / 4), 256, 0, st, p, (const float4*)dy, (const int4*)idx_max, (float4*)dx);  \
            else launch_pdl(pool_bwd_v4_kernel<MAXF, IDXT, false>, ew_blocks(total / 4), 256, 0, st, p, (const float4*)dy, (const int4*)idx_max, (float4*)dx);     \
        } while (0)
        if (is_max && unit && p.kh == 3 && p.kw == 3 && p.vstr == 2 && p.hstr == 2 && (int64_t)p.n * p.h <= 65535 &&
            (int64_t)p.w * (p.c / 4) < 0x7fffffffLL) {
            launch_pdl(pool_bwd_max_k3s2_kernel, dim3((unsigned)((p.w * (p.c / 4) + 255) / 256), (unsigned)(p.n * p.h)), 256, 0, st, p,
                       (const float4*)dy, (const int4*)idx_max, (float4*)dx);
            return check_launch("pool_bwd_max_k3s2");
        }
        if (is_max && small) B2C_POOL_BWD_V4(true, int);
        else if (is_max) B2C_POOL_BWD_V4(true, int64_t);
        else if (small) B2C_POOL_BWD_V4(false, int);
        else B2C_POOL_BWD_V4(false, int64_t);
#undef B2C_POOL_BWD_V4
        return check_launch("pool_backward_v4");
    }
    if (dtype == B2C_F32) {
        if (is_max) launch_pdl(pool_bwd_kernel<float, true>, ew_blocks(total), 256, 0, st, p, (const float*)dy, idx_max, (float*)dx, nchw);
        else launch_pdl(pool_bwd_kernel<float, false>, ew_blocks(total), 256, 0, st, p, (const float*)dy, idx_max, (float*)dx, nchw);
    } else {
        if (is_max) launch_pdl(pool_bwd_kernel<double, true>, ew_blocks(total), 256, 0, st, p, (const double*)dy, idx_max, (double*)dx, nchw);
        else launch_pdl(pool_bwd_kernel<double, false>, ew_blocks(total), 256, 0, st, p, (const double*)dy, idx_max, (double*)dx, nchw);
    }
    return check_launch("pool_backward");
}

extern "C" int b2c_softmax_forward(int dtype, int rows, int cols, const void* x, void* y, void* stream)
{
    CHECK_DTYPE(dtype);
    if (!x || !y) return B2C_ERR_NULL_POINTER;
    if (rows <= 0 || cols <= 0) return B2C_ERR_BAD_GEOMETRY;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == B2C_F32) launch_pdl(softmax_fwd_kernel<float>, rows, 256, 0, st, (const float*)x, (float*)y, cols);
    else launch_pdl(softmax_fwd_kernel<double>, rows, 256, 0, st, (const double*)x, (double*)y, cols);
    return check_launch("softmax_forward");
}

extern "C" int b2c_softmax_backward(int dtype, int rows, int cols, const void* dy, const void* y, void* dx, void* stream)
{
    CHECK_DTYPE(dtype);
    if (!dy || !y || !dx) return B2C_ERR_NULL_POINTER;
    if (rows <= 0 || cols <= 0) return B2C_ERR_BAD_GEOMETRY;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == B2C_F32) launch_pdl(softmax_bwd_kernel<float>, rows, 256, 0, st, (const float*)dy, (const float*)y, (float*)dx, cols);
    else launch_pdl(softmax_bwd_kernel<double>, rows, 256, 0, st, (const double*)dy, (const double*)y, (double*)dx, cols);
    return check_launch("softmax_backward");
}

extern "C" int b2c_cce_forward_backward(int dtype, int rows, int cols, const void* probs, const int32_t* labels,
                                        int global_batch, double eps, void* row_loss, int32_t* hit, void* dx, void* stream)
{
    CHECK_DTYPE(dtype);
    if (!probs || !labels || !row_loss || !dx) return B2C_ERR_NULL_POINTER;
    if (rows <= 0 || cols <= 0 || global_batch <= 0) return B2C_ERR_BAD_GEOMETRY;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == B2C_F32) launch_pdl(cce_kernel<float>, rows, 256, 0, st, (const float*)probs, labels, cols, global_batch, (float)eps, (float*)row_loss, hit, (float*)dx);
    else launch_pdl(cce_kernel<double>, rows, 256, 0, st, (const double*)probs, labels, cols, global_batch, eps, (double*)row_loss, hit, (double*)dx);
    return check_launch("cce");
}

extern "C" int b2c_cce_totals(int dtype, int rows, const void* row_loss, const int32_t* hit, double* out2, void* stream)
{
    CHECK_DTYPE(dtype);
    if (!row_loss || !out2) return B2C_ERR_NULL_POINTER;
    if (rows <= 0) return B2C_ERR_BAD_GEOMETRY;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == B2C_F32) launch_pdl(cce_totals_kernel<float>, 1, 256, 0, st, (const float*)row_loss, hit, rows, out2);
    else launch_pdl(cce_totals_kernel<double>, 1, 256, 0, st, (const double*)row_loss, hit, rows, out2);
    return check_launch("cce_totals");
}

extern "C" int b2c_bn_inv_std(int dtype, int c, const void* running_var, double eps, void* inv_std, void* stream)
{
    CHECK_DTYPE(dtype);
    if (!running_var || !inv_std) return B2C_ERR_NULL_POINTER;
    if (c <= 0) return B2C_ERR_BAD_GEOMETRY;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == B2C_F32) launch_pdl(bn_inv_std_kernel<float>, (c + 127) / 128, 128, 0, st, (const float*)running_var, c, eps, (float*)inv_std);
    else launch_pdl(bn_inv_std_kernel<double>, (c + 127) / 128, 128, 0, st, (const double*)running_var, c, eps, (double*)inv_std);
    return check_launch("bn_inv_std");
}

extern "C" int b2c_probe_fma(int dtype, int blocks, int iters, void* sink, double* flops, void* stream)
{
    CHECK_DTYPE(dtype);
    if (!sink) return B2C_ERR_NULL_POINTER;
    if (blocks <= 0 || iters <= 0) return B2C_ERR_BAD_GEOMETRY;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == B2C_F32) launch_pdl(fma_probe_kernel<float>, blocks, 256, 0, st, iters, 1.0f, (float*)sink);
    else launch_pdl(fma_probe_kernel<double>, blocks, 256, 0, st, iters, 1.0, (double*)sink);
    if (flops) *flops = 2.0 * 8.0 * 256.0 * (double)blocks * (double)iters;
    return check_launch("fma_probe");
}

extern "C" int b2c_sgd_update(int dtype, int64_t count, void* w, const void* dw, void* velocity,
                              double lr, double momentum, double decay, int nesterov, void* stream)
{
    CHECK_DTYPE(dtype);
    if (!w || !dw || !velocity) return B2C_ERR_NULL_POINTER;
    if (count < 0) return B2C_ERR_BAD_GEOMETRY;
    if (count == 0) return B2C_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == B2C_F32 && count % 4 == 0 && !(((uintptr_t)w | (uintptr_t)dw | (uintptr_t)velocity) & 15))
        launch_pdl(sgd_f4_kernel, ew_blocks(count / 8), 256, 0, st, (float4*)w, (const float4*)dw, (float4*)velocity, count / 4, (float)lr, (float)momentum,
                   (float)decay, nesterov);
    else if (dtype == B2C_F32) launch_pdl(sgd_kernel<float>, ew_blocks(count), 256, 0, st, (float*)w, (const float*)dw, (float*)velocity, count, (float)lr, (float)momentum, (float)decay, nesterov);
    else launch_pdl(sgd_kernel<double>, ew_blocks(count), 256, 0, st, (double*)w, (const double*)dw, (double*)velocity, count, lr, momentum, decay, nesterov);
    return check_launch("sgd_update");
}

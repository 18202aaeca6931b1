// HBM-bound layers either side of the convolution in a training step: batch normalisation,
// ReLU, residual sum, pooling, softmax, categorical cross-entropy and SGD.  All are single-pass
// streaming kernels over NHWC (rows, c) or NCHW (n, c, hw) tensors; per-channel reductions are
// two-stage with double partial sums so the result does not depend on launch order.
#include "b2c_common.cuh"
#include <float.h>

namespace b2c {

#define RED_CHUNKS 64

// ---- two-value per-channel reduction ---------------------------------------------------------
// F(flat_index, channel) -> (v0, v1); partial[chunk][2][c] in double.
template <typename F>
__global__ void reduce2_nhwc_kernel(F f, double* __restrict__ partial, int64_t rows, int c)
{
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
        reduce2_nhwc_kernel<F><<<grid, block, 0, st>>>(f, partial, rows, c);
    } else {
        dim3 grid(c, chunks);
        reduce2_nchw_kernel<F><<<grid, 256, 0, st>>>(f, partial, n, c, hw);
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
                                int64_t total, int c, int hw, int nchw, int relu, int ref_order)
{
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        int ch = channel_of(i, c, hw, nchw);
        T xn = (x[i] - mean[ch]) * inv_std[ch];
        T v = ref_order ? (xn * gamma[ch] + beta[ch]) : (gamma[ch] * xn + beta[ch]);
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
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        int ch = channel_of(i, c, hw, nchw);
        T g = dy[i];
        if (relu && !(y[i] > T(0))) g = T(0);
        T xn = (x[i] - mean[ch]) * inv_std[ch];
        dx[i] = (gamma[ch] * inv_std[ch] / count) * (count * g - xn * dgamma[ch] - dbeta[ch]);
    }
}

static unsigned ew_blocks(int64_t total) { int64_t b = (total + 255) / 256; return (unsigned)(b > 148 * 16 ? 148 * 16 : (b < 1 ? 1 : b)); }

template <typename T>
static int bn_train_forward_t(int layout, int n, int c, int hw, const T* x, const T* gamma, const T* beta,
                              T* rm, T* rv, double momentum, double eps, int relu, T* y, T* sm, T* si,
                              double* scratch, cudaStream_t st)
{
    int chunks;
    StatF<T> f{x};
    int rc = launch_reduce2(f, scratch, layout, n, c, hw, chunks, st);
    if (rc) return rc;
    bn_stats_final_kernel<T><<<(c + 127) / 128, 128, 0, st>>>(scratch, chunks, c, (double)n * hw, momentum, eps, rm, rv, sm, si);
    rc = check_launch("bn_stats_final"); if (rc) return rc;
    int64_t total = (int64_t)n * c * hw;
    bn_apply_kernel<T><<<ew_blocks(total), 256, 0, st>>>(x, y, sm, si, gamma, beta, total, c, hw, layout == B2C_LAYOUT_NCHW, relu, 0);
    return check_launch("bn_apply");
}

template <typename T>
static int bn_train_backward_t(int layout, int n, int c, int hw, const T* x, const T* dy, const T* y, const T* gamma,
                               const T* sm, const T* si, T* dgamma, T* dbeta, T* dx, double* scratch, cudaStream_t st)
{
    int chunks;
    int relu = y != nullptr;
    BnBwdF<T> f{x, dy, y, sm, si, relu};
    int rc = launch_reduce2(f, scratch, layout, n, c, hw, chunks, st);
    if (rc) return rc;
    bn_bwd_final_kernel<T><<<(c + 127) / 128, 128, 0, st>>>(scratch, chunks, c, dgamma, dbeta);
    rc = check_launch("bn_bwd_final"); if (rc) return rc;
    if (!dx) return B2C_OK;
    int64_t total = (int64_t)n * c * hw;
    bn_bwd_dx_kernel<T><<<ew_blocks(total), 256, 0, st>>>(x, dy, y, gamma, sm, si, dgamma, dbeta, dx, total, c, hw,
                                                          layout == B2C_LAYOUT_NCHW, relu, (T)((double)n * hw));
    return check_launch("bn_bwd_dx");
}

// ---- elementwise ---------------------------------------------------------------------------

template <typename T> __global__ void relu_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t n)
{
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) { T v = x[i]; y[i] = v > T(0) ? v : T(0); }
}
template <typename T> __global__ void relu_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ y, T* __restrict__ dx, int64_t n)
{
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dx[i] = y[i] > T(0) ? dy[i] : T(0);
}
template <typename T> __global__ void add_kernel(T* __restrict__ acc, const T* __restrict__ o, int64_t n)
{
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) acc[i] += o[i];
}
// float4 variants for the common aligned float32 case
__global__ void relu_fwd_f4_kernel(const float4* __restrict__ x, float4* __restrict__ y, int64_t n4)
{
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 v = x[i]; v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f); y[i] = v;
    }
}
__global__ void relu_bwd_f4_kernel(const float4* __restrict__ dy, const float4* __restrict__ y, float4* __restrict__ dx, int64_t n4)
{
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 g = dy[i], v = y[i];
        g.x = v.x > 0.f ? g.x : 0.f; g.y = v.y > 0.f ? g.y : 0.f; g.z = v.z > 0.f ? g.z : 0.f; g.w = v.w > 0.f ? g.w : 0.f;
        dx[i] = g;
    }
}
__global__ void add_f4_kernel(float4* __restrict__ acc, const float4* __restrict__ o, int64_t n4)
{
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

// ---- pooling -----------------------------------------------------------------------------------

struct PoolP {
    int n, h, w, c, ho, wo, kh, kw, vpad, hpad, vstr, hstr, vdil, hdil;
    int64_t xsn, xsh, xsw, xsc, ysn, ysh, ysw, ysc;
};

template <typename T, bool IS_MAX>
__global__ void pool_fwd_kernel(PoolP p, const T* __restrict__ x, T* __restrict__ y, int32_t* __restrict__ idx_max, int nchw)
{
    int64_t total = (int64_t)p.n * p.ho * p.wo * p.c;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        int cc, yy, xx, nn;
        if (nchw) { yy = (int)(i % p.wo); int64_t r = i / p.wo; xx = (int)(r % p.ho); r /= p.ho; cc = (int)(r % p.c); nn = (int)(r / p.c); }
        else { cc = (int)(i % p.c); int64_t r = i / p.c; yy = (int)(r % p.wo); r /= p.wo; xx = (int)(r % p.ho); nn = (int)(r / p.ho); }
        T best = IS_MAX ? (sizeof(T) == 4 ? (T)(-FLT_MAX) : (T)(-DBL_MAX)) : T(0);
        int bidx = 0, items = 0;
        for (int ii = 0; ii < p.kh; ii++) {
            int x_x = p.vstr * xx + p.vdil * ii - p.vpad;
            if (x_x < 0 || x_x >= p.h) continue;
            for (int jj = 0; jj < p.kw; jj++) {
                int x_y = p.hstr * yy + p.hdil * jj - p.hpad;
                if (x_y < 0 || x_y >= p.w) continue;
                T v = x[nn * p.xsn + x_x * p.xsh + x_y * p.xsw + cc * p.xsc];
                if (IS_MAX) { if (v > best) { best = v; bidx = ii * p.kw + jj; } }
                else { best += v; items++; }
            }
        }
        if (IS_MAX) { y[i] = best; if (idx_max) idx_max[i] = bidx; }
        else y[i] = best / (T)items;
    }
}

// Backward as a gather over the windows that contain each input element (fixed summation order).
template <typename T, bool IS_MAX>
__global__ void pool_bwd_kernel(PoolP p, const T* __restrict__ dy, const int32_t* __restrict__ idx_max, T* __restrict__ dx, int nchw)
{
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
                                         (float*)running_var, momentum, eps, fuse_relu, (float*)y, (float*)save_mean, (float*)save_inv_std, (double*)scratch, st);
    return bn_train_forward_t<double>(layout, n, c, hw, (const double*)x, (const double*)gamma, (const double*)beta, (double*)running_mean,
                                      (double*)running_var, momentum, eps, fuse_relu, (double*)y, (double*)save_mean, (double*)save_inv_std, (double*)scratch, st);
}

extern "C" int b2c_bn_train_backward(int dtype, int layout, int n, int c, int hw, const void* x, const void* dy,
                                     const void* y_for_relu_mask, const void* gamma, const void* save_mean,
                                     const void* save_inv_std, void* dgamma, void* dbeta, void* dx,
                                     void* scratch, size_t scratch_bytes, void* stream)
{
    CHECK_DTYPE(dtype); CHECK_LAYOUT(layout);
    if (!x || !dy || !gamma || !save_mean || !save_inv_std || !dgamma || !dbeta || !scratch) return B2C_ERR_NULL_POINTER;
    if (n <= 0 || c <= 0 || hw <= 0) return B2C_ERR_BAD_GEOMETRY;
    if (scratch_bytes < reduce2_bytes(c)) return B2C_ERR_WORKSPACE_TOO_SMALL;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == B2C_F32)
        return bn_train_backward_t<float>(layout, n, c, hw, (const float*)x, (const float*)dy, (const float*)y_for_relu_mask, (const float*)gamma,
                                          (const float*)save_mean, (const float*)save_inv_std, (float*)dgamma, (float*)dbeta, (float*)dx, (double*)scratch, st);
    return bn_train_backward_t<double>(layout, n, c, hw, (const double*)x, (const double*)dy, (const double*)y_for_relu_mask, (const double*)gamma,
                                       (const double*)save_mean, (const double*)save_inv_std, (double*)dgamma, (double*)dbeta, (double*)dx, (double*)scratch, st);
}

extern "C" int b2c_bn_inference(int dtype, int layout, int n, int c, int hw, const void* x, const void* mean,
                                const void* inv_std, const void* gamma, const void* beta, int relu, void* y, void* stream)
{
    CHECK_DTYPE(dtype); CHECK_LAYOUT(layout);
    if (!x || !mean || !inv_std || !gamma || !beta || !y) return B2C_ERR_NULL_POINTER;
    if (n <= 0 || c <= 0 || hw <= 0) return B2C_ERR_BAD_GEOMETRY;
    cudaStream_t st = (cudaStream_t)stream;
    int64_t total = (int64_t)n * c * hw;
    if (dtype == B2C_F32)
        bn_apply_kernel<float><<<ew_blocks(total), 256, 0, st>>>((const float*)x, (float*)y, (const float*)mean, (const float*)inv_std,
                                                                (const float*)gamma, (const float*)beta, total, c, hw, layout == B2C_LAYOUT_NCHW, relu, 1);
    else
        bn_apply_kernel<double><<<ew_blocks(total), 256, 0, st>>>((const double*)x, (double*)y, (const double*)mean, (const double*)inv_std,
                                                                 (const double*)gamma, (const double*)beta, total, c, hw, layout == B2C_LAYOUT_NCHW, relu, 1);
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
        if (f4_ok(count, x, y, y)) relu_fwd_f4_kernel<<<ew_blocks(count / 4), 256, 0, st>>>((const float4*)x, (float4*)y, count / 4);
        else relu_fwd_kernel<float><<<ew_blocks(count), 256, 0, st>>>((const float*)x, (float*)y, count);
    } else relu_fwd_kernel<double><<<ew_blocks(count), 256, 0, st>>>((const double*)x, (double*)y, count);
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
        if (f4_ok(count, dy, y, dx)) relu_bwd_f4_kernel<<<ew_blocks(count / 4), 256, 0, st>>>((const float4*)dy, (const float4*)y, (float4*)dx, count / 4);
        else relu_bwd_kernel<float><<<ew_blocks(count), 256, 0, st>>>((const float*)dy, (const float*)y, (float*)dx, count);
    } else relu_bwd_kernel<double><<<ew_blocks(count), 256, 0, st>>>((const double*)dy, (const double*)y, (double*)dx, count);
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
        if (f4_ok(count, acc, other, acc)) add_f4_kernel<<<ew_blocks(count / 4), 256, 0, st>>>((float4*)acc, (const float4*)other, count / 4);
        else add_kernel<float><<<ew_blocks(count), 256, 0, st>>>((float*)acc, (const float*)other, count);
    } else add_kernel<double><<<ew_blocks(count), 256, 0, st>>>((double*)acc, (const double*)other, count);
    return check_launch("add_inplace");
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
    if (dtype == B2C_F32) {
        if (is_max) pool_fwd_kernel<float, true><<<ew_blocks(total), 256, 0, st>>>(p, (const float*)x, (float*)y, idx_max, nchw);
        else pool_fwd_kernel<float, false><<<ew_blocks(total), 256, 0, st>>>(p, (const float*)x, (float*)y, idx_max, nchw);
    } else {
        if (is_max) pool_fwd_kernel<double, true><<<ew_blocks(total), 256, 0, st>>>(p, (const double*)x, (double*)y, idx_max, nchw);
        else pool_fwd_kernel<double, false><<<ew_blocks(total), 256, 0, st>>>(p, (const double*)x, (double*)y, idx_max, nchw);
    }
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
    if (dtype == B2C_F32) {
        if (is_max) pool_bwd_kernel<float, true><<<ew_blocks(total), 256, 0, st>>>(p, (const float*)dy, idx_max, (float*)dx, nchw);
        else pool_bwd_kernel<float, false><<<ew_blocks(total), 256, 0, st>>>(p, (const float*)dy, idx_max, (float*)dx, nchw);
    } else {
        if (is_max) pool_bwd_kernel<double, true><<<ew_blocks(total), 256, 0, st>>>(p, (const double*)dy, idx_max, (double*)dx, nchw);
        else pool_bwd_kernel<double, false><<<ew_blocks(total), 256, 0, st>>>(p, (const double*)dy, idx_max, (double*)dx, nchw);
    }
    return check_launch("pool_backward");
}

extern "C" int b2c_softmax_forward(int dtype, int rows, int cols, const void* x, void* y, void* stream)
{
    CHECK_DTYPE(dtype);
    if (!x || !y) return B2C_ERR_NULL_POINTER;
    if (rows <= 0 || cols <= 0) return B2C_ERR_BAD_GEOMETRY;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == B2C_F32) softmax_fwd_kernel<float><<<rows, 256, 0, st>>>((const float*)x, (float*)y, cols);
    else softmax_fwd_kernel<double><<<rows, 256, 0, st>>>((const double*)x, (double*)y, cols);
    return check_launch("softmax_forward");
}

extern "C" int b2c_softmax_backward(int dtype, int rows, int cols, const void* dy, const void* y, void* dx, void* stream)
{
    CHECK_DTYPE(dtype);
    if (!dy || !y || !dx) return B2C_ERR_NULL_POINTER;
    if (rows <= 0 || cols <= 0) return B2C_ERR_BAD_GEOMETRY;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == B2C_F32) softmax_bwd_kernel<float><<<rows, 256, 0, st>>>((const float*)dy, (const float*)y, (float*)dx, cols);
    else softmax_bwd_kernel<double><<<rows, 256, 0, st>>>((const double*)dy, (const double*)y, (double*)dx, cols);
    return check_launch("softmax_backward");
}

extern "C" int b2c_cce_forward_backward(int dtype, int rows, int cols, const void* probs, const int32_t* labels,
                                        int global_batch, double eps, void* row_loss, int32_t* hit, void* dx, void* stream)
{
    CHECK_DTYPE(dtype);
    if (!probs || !labels || !row_loss || !dx) return B2C_ERR_NULL_POINTER;
    if (rows <= 0 || cols <= 0 || global_batch <= 0) return B2C_ERR_BAD_GEOMETRY;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == B2C_F32) cce_kernel<float><<<rows, 256, 0, st>>>((const float*)probs, labels, cols, global_batch, (float)eps, (float*)row_loss, hit, (float*)dx);
    else cce_kernel<double><<<rows, 256, 0, st>>>((const double*)probs, labels, cols, global_batch, eps, (double*)row_loss, hit, (double*)dx);
    return check_launch("cce");
}

extern "C" int b2c_sgd_update(int dtype, int64_t count, void* w, const void* dw, void* velocity,
                              double lr, double momentum, double decay, int nesterov, void* stream)
{
    CHECK_DTYPE(dtype);
    if (!w || !dw || !velocity) return B2C_ERR_NULL_POINTER;
    if (count < 0) return B2C_ERR_BAD_GEOMETRY;
    if (count == 0) return B2C_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == B2C_F32) sgd_kernel<float><<<ew_blocks(count), 256, 0, st>>>((float*)w, (const float*)dw, (float*)velocity, count, (float)lr, (float)momentum, (float)decay, nesterov);
    else sgd_kernel<double><<<ew_blocks(count), 256, 0, st>>>((double*)w, (const double*)dw, (double*)velocity, count, lr, momentum, decay, nesterov);
    return check_launch("sgd_update");
}

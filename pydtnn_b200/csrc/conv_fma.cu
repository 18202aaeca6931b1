// Generic FMA engine: implicit-GEMM convolution (fprop / dgrad / wgrad) for float32 and float64,
// NHWC and NCHW, any filter layout, stride, padding and dilation.  The lowered matrix is never
// written to memory: each CTA gathers its A tile straight from the activation tensor using the
// same tap arithmetic the index-map kernel exposes for the bit-exact check.
//
//   fprop : C[pixel(n,ho,wo)][co] = sum_tap  x[pixel + tap] * w[co][tap]
//   dgrad : C[pixel(n,h,w)][ci]   = sum_tap  dy[(pixel + pad - tap) / stride] * w[tap.co][ci][tap.r][tap.s]
//   wgrad : C[tap(ci,r,s)][co]    = sum_pixel x[pixel + tap] * dy[pixel][co]      (split over pixels)
//
// float32 uses FP32 FMA, float64 uses FP64 FMA.  This engine is the one every shape can run on;
// the tensor-core engine (conv_tc.cu) takes over the shapes it supports.
#include "b2c_common.cuh"

namespace b2c {

enum { MODE_FPROP = 0, MODE_DGRAD = 1, MODE_WGRAD = 2 };

// Decoded pixel or tap. For a pixel: a_off = image base in the gathered tensor, (d0,d1) = the
// pixel's origin in gathered coordinates, b_off = its offset in the pixel-indexed second tensor.
// For a tap: a_off = channel offset, (d0,d1) = (r*vdil, s*hdil), b_off = offset in the filter tensor.
struct Info { int64_t a_off; int64_t b_off; int d0, d1; };

#define B2C_SENTINEL (1 << 29)

struct IgemmParams {
    int M, N, K;
    int P, Q, PQ;                 // pixel grid the pixel index runs over
    int C, R, S, tap_c_fast;      // tap space; tap_c_fast: index = (r*S+s)*C + c, else (c*R + r)*S + s
    int H, W;                     // extent of the gathered tensor
    int64_t a_sn, a_sh, a_sw, a_sc;
    int vstr, hstr, vpad, hpad, vdil, hdil;
    int64_t pb_sn, pb_sh, pb_sw;  // b_off of a pixel
    int64_t tb_sc, tb_sr, tb_ss;  // b_off of a tap
    int64_t b_sn;                 // B(k, n) = Bsrc[kinfo.b_off + n*b_sn]
    int64_t c_sn;                 // C(m, n) = Cdst[rowinfo.b_off + n*c_sn]
    int a_lanes_k, b_lanes_k;     // which index runs fastest across lanes when loading A / B
    int k_chunk, splits;
    int relu;
    // Sub-lattices (strided dgrad runs one launch per residue class of the output pixels, each with the taps that
    // reach it): pixel (pp, qq) of the grid is row pix_h0 + pp*pix_hs, column pix_w0 + qq*pix_ws of the tensor;
    // tap (r, s) of the (R, S) grid is filter tap (tap_r0 + r*tap_rs, tap_s0 + s*tap_ss).  Identity elsewhere.
    int pix_h0, pix_hs, pix_w0, pix_ws;
    int tap_r0, tap_rs, tap_s0, tap_ss;
};

template <typename T> struct Epilogue { const T *bias, *mean, *inv_std, *gamma, *beta; int relu; };

template <int MODE> __device__ __forceinline__ Info decode_pix(const IgemmParams& p, int idx, int limit) {
    Info f;
    if (idx >= limit) { f.a_off = 0; f.b_off = 0; f.d0 = -B2C_SENTINEL; f.d1 = 0; return f; }
    int n = idx / p.PQ; int rem = idx - n * p.PQ; int pp = rem / p.Q; int qq = rem - pp * p.Q;
    pp = p.pix_h0 + pp * p.pix_hs; qq = p.pix_w0 + qq * p.pix_ws;
    f.a_off = (int64_t)n * p.a_sn;
    f.b_off = (int64_t)n * p.pb_sn + (int64_t)pp * p.pb_sh + (int64_t)qq * p.pb_sw;
    if (MODE == MODE_DGRAD) { f.d0 = pp + p.vpad; f.d1 = qq + p.hpad; }
    else { f.d0 = pp * p.vstr - p.vpad; f.d1 = qq * p.hstr - p.hpad; }
    return f;
}

template <int MODE> __device__ __forceinline__ Info decode_tap(const IgemmParams& p, int idx, int limit) {
    Info f;
    if (idx >= limit) { f.a_off = 0; f.b_off = 0; f.d0 = (MODE == MODE_DGRAD) ? B2C_SENTINEL : -B2C_SENTINEL; f.d1 = 0; return f; }
    int c, r, s;
    if (p.tap_c_fast) { c = idx % p.C; int rs = idx / p.C; r = rs / p.S; s = rs - r * p.S; }
    else { int RS = p.R * p.S; c = idx / RS; int rs = idx - c * RS; r = rs / p.S; s = rs - r * p.S; }
    r = p.tap_r0 + r * p.tap_rs; s = p.tap_s0 + s * p.tap_ss;
    f.a_off = (int64_t)c * p.a_sc;
    f.b_off = (int64_t)c * p.tb_sc + (int64_t)r * p.tb_sr + (int64_t)s * p.tb_ss;
    f.d0 = r * p.vdil; f.d1 = s * p.hdil;
    return f;
}

__device__ __forceinline__ bool info_valid(const Info& f) { return f.d0 > -(B2C_SENTINEL >> 1) && f.d0 < (B2C_SENTINEL >> 1); }

// The tap arithmetic shared by every pass and by the index-map kernel: where in the gathered
// tensor does (pixel, tap) read, and is that inside the tensor?
template <int MODE>
__device__ __forceinline__ bool gather_off(const IgemmParams& p, const Info& pix, const Info& tap, int64_t& off) {
    int ih, iw;
    if (MODE == MODE_DGRAD) {
        int th = pix.d0 - tap.d0, tw = pix.d1 - tap.d1;
        if (th < 0 || tw < 0) return false;
        if (p.vstr != 1) { ih = th / p.vstr; if (ih * p.vstr != th) return false; } else ih = th;
        if (p.hstr != 1) { iw = tw / p.hstr; if (iw * p.hstr != tw) return false; } else iw = tw;
    } else {
        ih = pix.d0 + tap.d0; iw = pix.d1 + tap.d1;
    }
    if ((unsigned)ih >= (unsigned)p.H || (unsigned)iw >= (unsigned)p.W) return false;
    off = pix.a_off + tap.a_off + (int64_t)ih * p.a_sh + (int64_t)iw * p.a_sw;
    return true;
}

template <typename T> __device__ __forceinline__ void lds4(const T* p, T (&o)[4]);
template <> __device__ __forceinline__ void lds4<float>(const float* p, float (&o)[4]) {
    float4 v = *reinterpret_cast<const float4*>(p); o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
}
template <> __device__ __forceinline__ void lds4<double>(const double* p, double (&o)[4]) {
    double2 a = *reinterpret_cast<const double2*>(p), b = *reinterpret_cast<const double2*>(p + 2);
    o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
}

template <typename T> __device__ __forceinline__ T apply_epilogue(T v, int n, const Epilogue<T>& ep) {
    if (ep.bias) v += ep.bias[n];
    if (ep.mean) { T t = (v - ep.mean[n]) * ep.inv_std[n]; v = t * ep.gamma[n] + ep.beta[n]; }
    if (ep.relu) v = v > T(0) ? v : T(0);
    return v;
}

template <typename T> struct TileCfg;
template <> struct TileCfg<float> { static constexpr int BK = 16; };
template <> struct TileCfg<double> { static constexpr int BK = 8; };

template <typename T, int MODE, int BN, int TN>
__global__ void __launch_bounds__(256)
igemm_kernel(IgemmParams p, const T* __restrict__ A, const T* __restrict__ B, T* __restrict__ C,
             T* __restrict__ partial, Epilogue<T> ep)
{
    pdl_prologue();
    constexpr int BM = 128, NT = 256, BK = TileCfg<T>::BK;
    constexpr int A_PER = BM * BK / NT, B_PER = BN * BK / NT;
    constexpr int PADW = 16 / sizeof(T);
    __shared__ __align__(16) T As[2][BK][BM + PADW];
    __shared__ __align__(16) T Bs[2][BK][BN + PADW];
    __shared__ Info rowinfo[BM];
    __shared__ Info kinfo[2][BK];

    const int tid = threadIdx.x;
    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
    const int kbeg = blockIdx.z * p.k_chunk;
    const int kend = min(p.K, kbeg + p.k_chunk);
    const int nslice = (kend - kbeg + BK - 1) / BK;

    if (tid < BM)
        rowinfo[tid] = (MODE == MODE_WGRAD) ? decode_tap<MODE>(p, m0 + tid, p.M) : decode_pix<MODE>(p, m0 + tid, p.M);
    if (tid >= BM && tid < BM + BK) {
        int k = kbeg + (tid - BM);
        kinfo[0][tid - BM] = (MODE == MODE_WGRAD) ? decode_pix<MODE>(p, k, kend) : decode_tap<MODE>(p, k, kend);
    }
    __syncthreads();

    T ra[A_PER], rb[B_PER];
    auto fetch = [&](int buf) {
#pragma unroll
        for (int i = 0; i < A_PER; i++) {
            int e = tid + i * NT;
            int k = p.a_lanes_k ? (e % BK) : (e / BM);
            int m = p.a_lanes_k ? (e / BK) : (e % BM);
            const Info& ri = rowinfo[m];
            const Info& ki = kinfo[buf][k];
            int64_t off;
            bool ok = (MODE == MODE_WGRAD) ? gather_off<MODE>(p, ki, ri, off) : gather_off<MODE>(p, ri, ki, off);
            ra[i] = ok ? A[off] : T(0);
        }
#pragma unroll
        for (int i = 0; i < B_PER; i++) {
            int e = tid + i * NT;
            int k = p.b_lanes_k ? (e % BK) : (e / BN);
            int n = p.b_lanes_k ? (e / BK) : (e % BN);
            const Info& ki = kinfo[buf][k];
            bool ok = info_valid(ki) && (n0 + n) < p.N;
            rb[i] = ok ? B[ki.b_off + (int64_t)(n0 + n) * p.b_sn] : T(0);
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int i = 0; i < A_PER; i++) {
            int e = tid + i * NT;
            int k = p.a_lanes_k ? (e % BK) : (e / BM);
            int m = p.a_lanes_k ? (e / BK) : (e % BM);
            As[buf][k][m] = ra[i];
        }
#pragma unroll
        for (int i = 0; i < B_PER; i++) {
            int e = tid + i * NT;
            int k = p.b_lanes_k ? (e % BK) : (e / BN);
            int n = p.b_lanes_k ? (e / BK) : (e % BN);
            Bs[buf][k][n] = rb[i];
        }
    };

    T acc[8][TN];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) acc[i][j] = T(0);

    const int tx = tid & 15, ty = tid >> 4;

    if (nslice > 0) {
        fetch(0);
        stash(0);
        if (tid < BK) {
            int k = kbeg + BK + tid;
            kinfo[1][tid] = (MODE == MODE_WGRAD) ? decode_pix<MODE>(p, k, kend) : decode_tap<MODE>(p, k, kend);
        }
    }
    __syncthreads();

    for (int s = 0; s < nslice; s++) {
        const int cur = s & 1;
        if (s + 1 < nslice) fetch(cur ^ 1);
#pragma unroll
        for (int k = 0; k < BK; k++) {
            T a[8], b[TN];
            T t4[4];
            lds4<T>(&As[cur][k][ty * 4], t4);
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = t4[i];
            lds4<T>(&As[cur][k][BM / 2 + ty * 4], t4);
#pragma unroll
            for (int i = 0; i < 4; i++) a[4 + i] = t4[i];
            if (sizeof(T) == 8) {
                // doubles: two columns per 16-byte load, column pairs 32 apart, so that the 16 lanes of a row of the
                // thread grid read consecutive 16-byte words (four columns per thread would stride them 32 bytes
                // apart: a 4-way bank conflict)
#pragma unroll
                for (int g = 0; g < TN / 2; g++) {
                    const double2 v = *reinterpret_cast<const double2*>(&Bs[cur][k][g * 32 + tx * 2]);
                    b[2 * g] = (T)v.x; b[2 * g + 1] = (T)v.y;
                }
            } else {
                lds4<T>(&Bs[cur][k][tx * 4], t4);
#pragma unroll
                for (int j = 0; j < 4; j++) b[j] = t4[j];
                if (TN == 8) {
                    lds4<T>(&Bs[cur][k][BN / 2 + tx * 4], t4);
#pragma unroll
                    for (int j = 0; j < 4; j++) b[(TN == 8 ? 4 : 0) + j] = t4[j];
                }
            }
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < TN; j++) acc[i][j] = fma(a[i], b[j], acc[i][j]);
        }
        if (s + 1 < nslice) {
            stash(cur ^ 1);
            if (tid < BK) {
                int k = kbeg + (s + 2) * BK + tid;
                kinfo[cur][tid] = (MODE == MODE_WGRAD) ? decode_pix<MODE>(p, k, kend) : decode_tap<MODE>(p, k, kend);
            }
        }
        __syncthreads();
    }

    // epilogue
#pragma unroll
    for (int i = 0; i < 8; i++) {
        int rl = (i < 4) ? (ty * 4 + i) : (BM / 2 + ty * 4 + i - 4);
        int m = m0 + rl;
        if (m >= p.M) continue;
        const int64_t row_off = rowinfo[rl].b_off;
#pragma unroll
        for (int j = 0; j < TN; j++) {
            int cl = sizeof(T) == 8 ? ((j >> 1) * 32 + tx * 2 + (j & 1)) : ((j < 4) ? (tx * 4 + j) : (BN / 2 + tx * 4 + j - 4));
            int n = n0 + cl;
            if (n >= p.N) continue;
            if (p.splits > 1) partial[((int64_t)blockIdx.z * p.M + m) * p.N + n] = acc[i][j];
            else C[row_off + (int64_t)n * p.c_sn] = apply_epilogue<T>(acc[i][j], n, ep);
        }
    }
}

// Second stage of split-K: fixed-order sum over the splits, epilogue, scatter to the output.
template <typename T, int MODE>
__global__ void splitk_reduce_kernel(IgemmParams p, const T* __restrict__ partial, T* __restrict__ C, Epilogue<T> ep)
{
    pdl_prologue();
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t total = (int64_t)p.M * p.N;
    if (idx >= total) return;
    int m = (int)(idx / p.N), n = (int)(idx - (int64_t)m * p.N);
    T v = T(0);
    for (int z = 0; z < p.splits; z++) v += partial[(int64_t)z * total + idx];
    Info ri = (MODE == MODE_WGRAD) ? decode_tap<MODE>(p, m, p.M) : decode_pix<MODE>(p, m, p.M);
    C[ri.b_off + (int64_t)n * p.c_sn] = apply_epilogue<T>(v, n, ep);
}

// Index map of the lowering, numbered as the reference numbers rows and columns.
__global__ void index_map_kernel(IgemmParams p, int64_t* __restrict__ map, int nchw)
{
    pdl_prologue();
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t total = (int64_t)p.M * p.K;
    if (idx >= total) return;
    int m, t;
    if (nchw) { t = (int)(idx / p.M); m = (int)(idx - (int64_t)t * p.M); }
    else { m = (int)(idx / p.K); t = (int)(idx - (int64_t)m * p.K); }
    Info pix = decode_pix<MODE_FPROP>(p, m, p.M);
    Info tap = decode_tap<MODE_FPROP>(p, t, p.K);
    int64_t off;
    bool ok = gather_off<MODE_FPROP>(p, pix, tap, off);
    map[idx] = ok ? off : -1;
}

// ---- fully connected layer: weight gradient as an outer-product sum ---------------------------------
// dw[i][o] = sum_b x[b][i] * dy[b][o] for a (batch, in) input, a (batch, out) output gradient and an (in, out)
// row-major weight matrix (pydtnn/backends/cpu/layers/fc_cpu.py:66-71).  The sum is over the batch only (32-64
// terms), so the pass is bound by writing dw; the general kernel above spends its time on gather arithmetic that a
// dense matrix does not need.  One CTA = one 128 x 128 tile of dw, all of the batch, 8 x 8 outputs per thread.
template <typename T> __device__ __forceinline__ void ldg4(const T* p, T (&o)[4]);
template <> __device__ __forceinline__ void ldg4<float>(const float* p, float (&o)[4]) {
    float4 v = __ldg(reinterpret_cast<const float4*>(p)); o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
}
template <> __device__ __forceinline__ void ldg4<double>(const double* p, double (&o)[4]) {
    double2 a = __ldg(reinterpret_cast<const double2*>(p)), b = __ldg(reinterpret_cast<const double2*>(p) + 1);
    o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
}
template <typename T> __device__ __forceinline__ void sts4(T* p, const T (&v)[4]);
template <> __device__ __forceinline__ void sts4<float>(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <> __device__ __forceinline__ void sts4<double>(double* p, const double (&v)[4]) {
    *reinterpret_cast<double2*>(p) = make_double2(v[0], v[1]); *reinterpret_cast<double2*>(p + 2) = make_double2(v[2], v[3]);
}

template <typename T>
__global__ void __launch_bounds__(256)
fc_wgrad_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ dw, int batch, int in_f, int out_f)
{
    pdl_prologue();
    constexpr int BT = 128, KC = TileCfg<T>::BK, PER = KC * BT / 4 / 256;     // 4-element vectors per thread per tile
    __shared__ __align__(16) T xs[2][KC][BT];
    __shared__ __align__(16) T ds[2][KC][BT];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int o0 = blockIdx.x * BT, i0 = blockIdx.y * BT;
    T rx[PER][4], rd[PER][4];
    auto fetch = [&](int b0) {
#pragma unroll
        for (int j = 0; j < PER; j++) {
            const int v = tid + j * 256, k = v / (BT / 4), col = (v % (BT / 4)) * 4;
            const bool row_ok = b0 + k < batch;
            if (row_ok && i0 + col < in_f) ldg4<T>(x + (int64_t)(b0 + k) * in_f + i0 + col, rx[j]);
            else { rx[j][0] = rx[j][1] = rx[j][2] = rx[j][3] = T(0); }
            if (row_ok && o0 + col < out_f) ldg4<T>(dy + (int64_t)(b0 + k) * out_f + o0 + col, rd[j]);
            else { rd[j][0] = rd[j][1] = rd[j][2] = rd[j][3] = T(0); }
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int j = 0; j < PER; j++) {
            const int v = tid + j * 256, k = v / (BT / 4), col = (v % (BT / 4)) * 4;
            sts4<T>(&xs[buf][k][col], rx[j]);
            sts4<T>(&ds[buf][k][col], rd[j]);
        }
    };
    T acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = T(0);
    const int nchunk = (batch + KC - 1) / KC;
    fetch(0);
    stash(0);
    __syncthreads();
    for (int c = 0; c < nchunk; c++) {
        const int cur = c & 1;
        if (c + 1 < nchunk) fetch((c + 1) * KC);
#pragma unroll
        for (int k = 0; k < KC; k++) {
            T a[8], b[8], t4[4];
            lds4<T>(&xs[cur][k][ty * 4], t4);
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = t4[i];
            lds4<T>(&xs[cur][k][BT / 2 + ty * 4], t4);
#pragma unroll
            for (int i = 0; i < 4; i++) a[4 + i] = t4[i];
            lds4<T>(&ds[cur][k][tx * 4], t4);
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = t4[j];
            lds4<T>(&ds[cur][k][BT / 2 + tx * 4], t4);
#pragma unroll
            for (int j = 0; j < 4; j++) b[4 + j] = t4[j];
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < 8; j++) acc[i][j] = fma(a[i], b[j], acc[i][j]);
        }
        if (c + 1 < nchunk) stash(cur ^ 1);
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int row = i0 + ((i < 4) ? (ty * 4 + i) : (BT / 2 + ty * 4 + i - 4));
        if (row >= in_f) continue;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int col = o0 + h * (BT / 2) + tx * 4;
            if (col >= out_f) continue;
            const T v[4] = {acc[i][4 * h], acc[i][4 * h + 1], acc[i][4 * h + 2], acc[i][4 * h + 3]};
            sts4<T>(dw + (int64_t)row * out_f + col, v);
        }
    }
}

static bool is_dense_fc(const Geo& g)
{
    return g.layout == B2C_LAYOUT_NHWC && g.w_layout == B2C_W_CRSK && g.h == 1 && g.w == 1 && g.kh == 1 && g.kw == 1 &&
           g.vpad == 0 && g.hpad == 0 && g.ci % 4 == 0 && g.co % 4 == 0;
}

// ---- host side ----------------------------------------------------------------------------

static IgemmParams make_params(const Geo& g, int mode)
{
    IgemmParams p{};
    ActStride xs = act_stride(g.layout, g.h, g.w, g.ci);
    ActStride ys = act_stride(g.layout, g.ho, g.wo, g.co);
    WStride ws = w_stride(g.w_layout, g.ci, g.co, g.kh, g.kw);
    const bool nhwc = g.layout == B2C_LAYOUT_NHWC;
    p.R = g.kh; p.S = g.kw;
    p.vstr = g.vstr; p.hstr = g.hstr; p.vpad = g.vpad; p.hpad = g.hpad; p.vdil = g.vdil; p.hdil = g.hdil;
    p.relu = 0; p.splits = 1;
    p.pix_h0 = 0; p.pix_hs = 1; p.pix_w0 = 0; p.pix_ws = 1;
    p.tap_r0 = 0; p.tap_rs = 1; p.tap_s0 = 0; p.tap_ss = 1;
    if (mode == MODE_FPROP) {
        p.M = (int)g.M; p.N = g.co; p.K = (int)g.K;
        p.P = g.ho; p.Q = g.wo; p.C = g.ci; p.H = g.h; p.W = g.w;
        p.a_sn = xs.sn; p.a_sh = xs.sh; p.a_sw = xs.sw; p.a_sc = xs.sc;
        p.pb_sn = ys.sn; p.pb_sh = ys.sh; p.pb_sw = ys.sw; p.c_sn = ys.sc;
        p.tb_sc = ws.sc; p.tb_sr = ws.sr; p.tb_ss = ws.ss; p.b_sn = ws.sk;
        p.tap_c_fast = nhwc; p.a_lanes_k = nhwc;
        p.b_lanes_k = (g.w_layout != B2C_W_CRSK);
    } else if (mode == MODE_DGRAD) {
        p.M = g.n * g.h * g.w; p.N = g.ci; p.K = g.co * g.kh * g.kw;
        p.P = g.h; p.Q = g.w; p.C = g.co; p.H = g.ho; p.W = g.wo;
        p.a_sn = ys.sn; p.a_sh = ys.sh; p.a_sw = ys.sw; p.a_sc = ys.sc;
        p.pb_sn = xs.sn; p.pb_sh = xs.sh; p.pb_sw = xs.sw; p.c_sn = xs.sc;
        p.tb_sc = ws.sk; p.tb_sr = ws.sr; p.tb_ss = ws.ss; p.b_sn = ws.sc;
        p.tap_c_fast = nhwc; p.a_lanes_k = nhwc;
        p.b_lanes_k = (g.w_layout != B2C_W_KRSC);
    } else {
        p.M = (int)g.K; p.N = g.co; p.K = (int)g.M;
        p.P = g.ho; p.Q = g.wo; p.C = g.ci; p.H = g.h; p.W = g.w;
        p.a_sn = xs.sn; p.a_sh = xs.sh; p.a_sw = xs.sw; p.a_sc = xs.sc;
        p.pb_sn = ys.sn; p.pb_sh = ys.sh; p.pb_sw = ys.sw; p.b_sn = ys.sc;
        p.tb_sc = ws.sc; p.tb_sr = ws.sr; p.tb_ss = ws.ss; p.c_sn = ws.sk;
        p.tap_c_fast = nhwc;          // rows run over taps: channel fastest keeps NHWC loads contiguous
        p.a_lanes_k = !nhwc;          // NCHW: pixels are contiguous
        p.b_lanes_k = !nhwc;
    }
    p.PQ = p.P * p.Q;
    return p;
}

static int tile_bn(int N) { return N <= 64 ? 64 : 128; }

// Number of K splits: enough CTAs to fill the 148 SMs about twice, each split at least 8 slices.
static int choose_splits(const IgemmParams& p, int bk)
{
    int64_t ctas = (int64_t)((p.M + 127) / 128) * ((p.N + tile_bn(p.N) - 1) / tile_bn(p.N));
    if (ctas >= 148) return 1;
    int64_t want = (296 + ctas - 1) / ctas;
    int64_t max_by_k = p.K / (8 * bk);
    if (max_by_k < 1) max_by_k = 1;
    int64_t s = want < max_by_k ? want : max_by_k;
    if (s > 128) s = 128;
    return (int)s;
}

static void finish_params(IgemmParams& p, int dtype)
{
    int bk = dtype == B2C_F32 ? 16 : 8;
    if (p.K <= 0) { p.splits = 1; p.k_chunk = bk; return; }        // no taps reach these pixels: the launch writes zeros
    p.splits = choose_splits(p, bk);
    int chunk = (p.K + p.splits - 1) / p.splits;
    chunk = (chunk + bk - 1) / bk * bk;
    p.k_chunk = chunk;
    p.splits = (p.K + chunk - 1) / chunk;
}

// Strided dgrad, dilation 1: input pixel (h, w) only receives taps with r = (h + vpad) mod vstr, s = (w + hpad) mod hstr
// (mod the strides).  Class (a, b) of those residues is a dense problem over its own pixels and taps; gathering all
// taps for all pixels instead would spend (vstr*hstr - 1) / (vstr*hstr) of the inner loop on zeros.
static bool dgrad_by_class(const Geo& g) { return (g.vstr > 1 || g.hstr > 1) && g.vdil == 1 && g.hdil == 1; }

static IgemmParams dgrad_class_params(const Geo& g, int a, int b)
{
    IgemmParams p = make_params(g, MODE_DGRAD);
    const int h0 = ((a - g.vpad) % g.vstr + g.vstr) % g.vstr, w0 = ((b - g.hpad) % g.hstr + g.hstr) % g.hstr;
    p.pix_h0 = h0; p.pix_hs = g.vstr; p.pix_w0 = w0; p.pix_ws = g.hstr;
    p.P = h0 < g.h ? (g.h - h0 + g.vstr - 1) / g.vstr : 0;
    p.Q = w0 < g.w ? (g.w - w0 + g.hstr - 1) / g.hstr : 0;
    p.PQ = p.P * p.Q;
    p.M = g.n * p.PQ;
    p.tap_r0 = a; p.tap_rs = g.vstr; p.tap_s0 = b; p.tap_ss = g.hstr;
    p.R = a < g.kh ? (g.kh - a + g.vstr - 1) / g.vstr : 0;
    p.S = b < g.kw ? (g.kw - b + g.hstr - 1) / g.hstr : 0;
    p.K = g.co * p.R * p.S;
    return p;
}

size_t fma_workspace_bytes(const Geo& g, int pass)
{
    size_t es = g.dtype == B2C_F32 ? 4 : 8;
    if (pass == B2C_PASS_DGRAD && dgrad_by_class(g)) {
        size_t most = 0;
        for (int a = 0; a < g.vstr; a++)
            for (int b = 0; b < g.hstr; b++) {
                IgemmParams p = dgrad_class_params(g, a, b);
                if (p.M == 0) continue;
                finish_params(p, g.dtype);
                size_t bytes = p.splits > 1 ? (size_t)p.splits * p.M * p.N * es : 0;
                if (bytes > most) most = bytes;
            }
        return most;
    }
    IgemmParams p = make_params(g, pass);
    finish_params(p, g.dtype);
    size_t bytes = p.splits > 1 ? (size_t)p.splits * p.M * p.N * es : 0;
    if (pass == B2C_PASS_WGRAD) bytes = align_up(bytes, 256) + channel_sum_workspace_bytes(g.n, g.co, g.ho * g.wo);
    return bytes;
}

template <typename T, int MODE>
static int launch_igemm(IgemmParams& p, const void* A, const void* B, void* C, void* ws, size_t ws_bytes,
                        Epilogue<T> ep, cudaStream_t st)
{
    finish_params(p, sizeof(T) == 4 ? B2C_F32 : B2C_F64);
    size_t need = p.splits > 1 ? (size_t)p.splits * p.M * p.N * sizeof(T) : 0;
    if (need > ws_bytes || (need && !ws)) return B2C_ERR_WORKSPACE_TOO_SMALL;
    const int bn = tile_bn(p.N);
    dim3 grid((p.M + 127) / 128, (p.N + bn - 1) / bn, p.splits);
    if (grid.y > 65535 || grid.z > 65535) return B2C_ERR_TOO_LARGE;
    if (bn == 64)
        launch_pdl(igemm_kernel<T, MODE, 64, 4>, grid, 256, 0, st, p, (const T*)A, (const T*)B, (T*)C, (T*)ws, ep);
    else
        launch_pdl(igemm_kernel<T, MODE, 128, 8>, grid, 256, 0, st, p, (const T*)A, (const T*)B, (T*)C, (T*)ws, ep);
    int rc = check_launch("igemm_kernel");
    if (rc) return rc;
    if (p.splits > 1) {
        int64_t total = (int64_t)p.M * p.N;
        launch_pdl(splitk_reduce_kernel<T, MODE>, (unsigned)((total + 255) / 256), 256, 0, st, p, (const T*)ws, (T*)C, ep);
        rc = check_launch("splitk_reduce_kernel");
    }
    return rc;
}

template <typename T>
static Epilogue<T> make_epilogue(const void* bias, const b2c_bn_params* bn, int relu)
{
    Epilogue<T> ep{};
    ep.bias = (const T*)bias;
    if (bn) { ep.mean = (const T*)bn->mean; ep.inv_std = (const T*)bn->inv_std; ep.gamma = (const T*)bn->gamma; ep.beta = (const T*)bn->beta; }
    ep.relu = relu;
    return ep;
}

int fma_fprop(const Geo& g, const void* x, const void* w, const void* bias, const b2c_bn_params* bn, int relu,
              void* y, void* ws, size_t ws_bytes, cudaStream_t st)
{
    IgemmParams p = make_params(g, MODE_FPROP);
    if (g.dtype == B2C_F32) return launch_igemm<float, MODE_FPROP>(p, x, w, y, ws, ws_bytes, make_epilogue<float>(bias, bn, relu), st);
    return launch_igemm<double, MODE_FPROP>(p, x, w, y, ws, ws_bytes, make_epilogue<double>(bias, bn, relu), st);
}

int fma_dgrad(const Geo& g, const void* dy, const void* w, void* dx, void* ws, size_t ws_bytes, cudaStream_t st)
{
    if (dgrad_by_class(g)) {
        for (int a = 0; a < g.vstr; a++)
            for (int b = 0; b < g.hstr; b++) {
                IgemmParams p = dgrad_class_params(g, a, b);
                if (p.M == 0) continue;
                int rc = g.dtype == B2C_F32
                    ? launch_igemm<float, MODE_DGRAD>(p, dy, w, dx, ws, ws_bytes, Epilogue<float>{}, st)
                    : launch_igemm<double, MODE_DGRAD>(p, dy, w, dx, ws, ws_bytes, Epilogue<double>{}, st);
                if (rc) return rc;
            }
        return B2C_OK;
    }
    IgemmParams p = make_params(g, MODE_DGRAD);
    if (g.dtype == B2C_F32) return launch_igemm<float, MODE_DGRAD>(p, dy, w, dx, ws, ws_bytes, Epilogue<float>{}, st);
    return launch_igemm<double, MODE_DGRAD>(p, dy, w, dx, ws, ws_bytes, Epilogue<double>{}, st);
}

int fma_wgrad(const Geo& g, const void* x, const void* dy, void* dw, void* db, void* ws, size_t ws_bytes,
              cudaStream_t st)
{
    const size_t align = g.dtype == B2C_F32 ? 15 : 31;
    if (is_dense_fc(g) && !(((uintptr_t)x | (uintptr_t)dy | (uintptr_t)dw) & align)) {
        dim3 grid((g.co + 127) / 128, (g.ci + 127) / 128);
        if (grid.y > 65535) return B2C_ERR_TOO_LARGE;
        if (g.dtype == B2C_F32) launch_pdl(fc_wgrad_kernel<float>, grid, 256, 0, st, (const float*)x, (const float*)dy, (float*)dw, g.n, g.ci, g.co);
        else launch_pdl(fc_wgrad_kernel<double>, grid, 256, 0, st, (const double*)x, (const double*)dy, (double*)dw, g.n, g.ci, g.co);
        int rc = check_launch("fc_wgrad_kernel");
        if (rc || !db) return rc;
        size_t cs = channel_sum_workspace_bytes(g.n, g.co, 1);
        if (!ws || ws_bytes < cs) return B2C_ERR_WORKSPACE_TOO_SMALL;
        return channel_sum(g.dtype, g.layout, g.n, g.co, 1, dy, db, ws, cs, st);
    }
    IgemmParams p = make_params(g, MODE_WGRAD);
    finish_params(p, g.dtype);
    size_t es = g.dtype == B2C_F32 ? 4 : 8;
    size_t part = align_up(p.splits > 1 ? (size_t)p.splits * p.M * p.N * es : 0, 256);
    int rc;
    if (g.dtype == B2C_F32) rc = launch_igemm<float, MODE_WGRAD>(p, x, dy, dw, ws, ws_bytes, Epilogue<float>{}, st);
    else rc = launch_igemm<double, MODE_WGRAD>(p, x, dy, dw, ws, ws_bytes, Epilogue<double>{}, st);
    if (rc || !db) return rc;
    size_t cs = channel_sum_workspace_bytes(g.n, g.co, g.ho * g.wo);
    if (!ws || ws_bytes < part + cs) return B2C_ERR_WORKSPACE_TOO_SMALL;
    return channel_sum(g.dtype, g.layout, g.n, g.co, g.ho * g.wo, dy, db, (char*)ws + part, cs, st);
}

int fma_index_map(const Geo& g, int64_t* map, cudaStream_t st)
{
    Geo gr = g;
    IgemmParams p = make_params(gr, MODE_FPROP);
    p.tap_c_fast = 0;  // the reference numbers taps channel-slowest: col = cc*kh*kw + ii*kw + jj
    int64_t total = (int64_t)p.M * p.K;
    if (total > (int64_t)0x7fffffff * 256) return B2C_ERR_TOO_LARGE;
    launch_pdl(index_map_kernel, (unsigned)((total + 255) / 256), 256, 0, st, p, map, g.layout == B2C_LAYOUT_NCHW);
    return check_launch("index_map_kernel");
}

// ---- per-channel sum (bias gradient) ----------------------------------------------------------

#define CS_CHUNKS 64

// NHWC: src is (rows, c). Block (32, 8): x runs over channels, y over rows of one chunk.
template <typename T>
__global__ void channel_sum_nhwc_kernel(const T* __restrict__ src, double* __restrict__ partial, int64_t rows, int c)
{
    pdl_prologue();
    __shared__ double sm[8][33];
    int ch = blockIdx.x * 32 + threadIdx.x;
    int64_t per = (rows + gridDim.y - 1) / gridDim.y;
    int64_t r0 = (int64_t)blockIdx.y * per, r1 = r0 + per < rows ? r0 + per : rows;
    double acc = 0.0;
    if (ch < c)
        for (int64_t r = r0 + threadIdx.y; r < r1; r += 8) acc += (double)src[r * c + ch];
    sm[threadIdx.y][threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.y == 0 && ch < c) {
        double s = 0.0;
        for (int i = 0; i < 8; i++) s += sm[i][threadIdx.x];
        partial[(int64_t)blockIdx.y * c + ch] = s;
    }
}

// NCHW: src is (n, c, hw). One block per (channel, chunk); threads stride over (image, position).
template <typename T>
__global__ void channel_sum_nchw_kernel(const T* __restrict__ src, double* __restrict__ partial, int n, int c, int hw)
{
    pdl_prologue();
    __shared__ double sm[256];
    int ch = blockIdx.x;
    int64_t total = (int64_t)n * hw;
    int64_t per = (total + gridDim.y - 1) / gridDim.y;
    int64_t i0 = (int64_t)blockIdx.y * per, i1 = i0 + per < total ? i0 + per : total;
    double acc = 0.0;
    for (int64_t i = i0 + threadIdx.x; i < i1; i += 256) {
        int64_t img = i / hw, pos = i - img * hw;
        acc += (double)src[(img * c + ch) * hw + pos];
    }
    sm[threadIdx.x] = acc;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) { if (threadIdx.x < s) sm[threadIdx.x] += sm[threadIdx.x + s]; __syncthreads(); }
    if (threadIdx.x == 0) partial[(int64_t)blockIdx.y * c + ch] = sm[0];
}

template <typename T>
__global__ void channel_sum_final_kernel(const double* __restrict__ partial, T* __restrict__ dst, int c, int chunks)
{
    pdl_prologue();
    int ch = blockIdx.x * blockDim.x + threadIdx.x;
    if (ch >= c) return;
    double s = 0.0;
    for (int i = 0; i < chunks; i++) s += partial[(int64_t)i * c + ch];
    dst[ch] = (T)s;
}

// Enough for the float4 fast path to spread over about four CTAs per SM: two doubles per channel and chunk.
size_t channel_sum_workspace_bytes(int n, int c, int hw)
{
    (void)n; (void)hw;
    int gx = c / 256 > 0 ? c / 256 : 1;
    int chunks = (592 + gx - 1) / gx;
    if (chunks < CS_CHUNKS) chunks = CS_CHUNKS;
    return (size_t)chunks * 2 * c * sizeof(double);
}

int channel_sum(int dtype, int layout, int n, int c, int hw, const void* src, void* dst, void* ws, size_t ws_bytes,
                cudaStream_t st)
{
    if (!src || !dst || !ws) return B2C_ERR_NULL_POINTER;
    if (ws_bytes < (size_t)CS_CHUNKS * c * sizeof(double)) return B2C_ERR_WORKSPACE_TOO_SMALL;
    if (dtype == B2C_F32 && layout == B2C_LAYOUT_NHWC) {
        int r = channel_sum_v4(n, c, hw, src, dst, ws, ws_bytes, st);
        if (r != 1) return r;     // 1 = fast path not applicable
    }
    double* partial = (double*)ws;
    int64_t rows = (int64_t)n * hw;
    int chunks = (int)(rows < CS_CHUNKS ? rows : CS_CHUNKS);
    if (chunks < 1) chunks = 1;
    if (layout == B2C_LAYOUT_NHWC) {
        dim3 grid((c + 31) / 32, chunks), block(32, 8);
        if (dtype == B2C_F32) launch_pdl(channel_sum_nhwc_kernel<float>, grid, block, 0, st, (const float*)src, partial, rows, c);
        else launch_pdl(channel_sum_nhwc_kernel<double>, grid, block, 0, st, (const double*)src, partial, rows, c);
    } else {
        if (c > 65535 * 32) return B2C_ERR_TOO_LARGE;
        dim3 grid(c, chunks);
        if (dtype == B2C_F32) launch_pdl(channel_sum_nchw_kernel<float>, grid, 256, 0, st, (const float*)src, partial, n, c, hw);
        else launch_pdl(channel_sum_nchw_kernel<double>, grid, 256, 0, st, (const double*)src, partial, n, c, hw);
    }
    int rc = check_launch("channel_sum");
    if (rc) return rc;
    if (dtype == B2C_F32) launch_pdl(channel_sum_final_kernel<float>, (c + 255) / 256, 256, 0, st, partial, (float*)dst, c, chunks);
    else launch_pdl(channel_sum_final_kernel<double>, (c + 255) / 256, 256, 0, st, partial, (double*)dst, c, chunks);
    return check_launch("channel_sum_final");
}

}  // namespace b2c

// Tensor-core engine for float32 NHWC convolutions on sm_100a: implicit GEMM on tcgen05 with
// accumulators in tensor memory, operands staged by TMA, float32 accuracy kept by a 3xTF32 split.
//
// The lowered (im2row) matrix never exists: the producer warp issues TMA *im2col-mode* loads that
// gather, for one filter tap and one block of 32 channels, the 128 consecutive output pixels of a
// tile straight into a 128B-swizzled K-major shared-memory tile (padding = TMA out-of-bounds
// zero fill, conv stride = TMA traversal stride).
//
//   fprop : y[pixel][co]  = sum_{tap,c} x[pixel+tap][c]  * w[co][tap][c]
//   dgrad : dx[pixel][ci] = sum_{tap,c} dy[pixel+tap'][c] * w[c][flip(tap')][ci]   (stride 1)
//           -- the same kernel run on dy with padding (k-1)*dil - pad and a flipped, transposed
//              filter copy
//   wgrad : dw[co][tap][ci] = sum_pixel x[pixel+tap][ci] * dy[pixel][co]           (split over pixels)
//
// 3xTF32: every float32 operand a is split as a = hi + lo with hi = tf32(a) (round to nearest) and
// lo = a - hi (exact in float32).  Three tensor-core products lo*hi + hi*lo + hi*hi accumulate in
// the float32 TMEM tile (small terms first).  Filters are split once per call by a small kernel;
// activation tiles are split in shared memory by the transform warps between TMA arrival and MMA
// issue.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2-5 = operand transform during the main loop, then epilogue (TMEM -> registers ->
// bias / BN-scale / ReLU -> global).  Every mbarrier wait is bounded: when a wait runs out the
// CTA raises an abort flag, records a status word in global memory, skips its remaining work,
// frees its tensor memory and returns.
#include "b2c_common.cuh"
#include <cuda.h>

namespace b2c {

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}

#define TC_WAIT_CYCLES 2000000000LL   // about one second at the boost clock

// Bounded wait. Returns false when the wait ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = clock64();
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > TC_WAIT_CYCLES) {
            *abort_flag = 1;
            atomicCAS(status, 0, code);
            return false;
        }
    }
}

__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_load_im2col_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c, int w, int h,
                                                   int n, uint16_t off_w, uint16_t off_h) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes"
                 " [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h)
                 : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], tf32 inputs, f32 accumulate.
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrive on an mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float to_tf32_rn(float v) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return __uint_as_float(r);
}

// Shared-memory matrix descriptor, 128-byte swizzle, rows of 128 bytes, 8-row groups 1024 bytes
// apart.  K-major: the 128-byte row is 32 K elements of one M/N row (leading offset unused).
// MN-major: the 128-byte row is 32 M/N elements of one K index; further 32-element groups lie
// `lbo_bytes` apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;     // descriptor version for sm_100
    d |= (uint64_t)2 << 61;     // SWIZZLE_128B
    return d;
}
// Instruction descriptor: tf32 x tf32 -> f32, dense.
__host__ __device__ constexpr uint32_t make_idesc_tf32(int M, int N, int a_mn_major, int b_mn_major) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// Device status word shared by all tensor-core kernels (0 = fine).
__device__ int g_tc_status = 0;

enum { TC_ERR_FULL = 1, TC_ERR_XFORM = 2, TC_ERR_EMPTY = 3, TC_ERR_ACCUM = 4 };

// ---------------------------------------------------------------------------------------------
// Filter preparation: hi/lo split into the K-major GEMM layout the kernels read through TMA
// ---------------------------------------------------------------------------------------------
struct PrepParams {
    int rows, C, R, S;          // output is [rows][(r*S+s)*C + c]
    int64_t s_row, s_c, s_r, s_s;  // element strides of the source filter by (row, c, r, s)
    int flip;                   // 1: read tap (R-1-r, S-1-s)
};

__global__ void tc_prep_filter_kernel(PrepParams p, const float* __restrict__ w, float* __restrict__ hi, float* __restrict__ lo)
{
    int64_t K = (int64_t)p.R * p.S * p.C;
    int64_t total = (int64_t)p.rows * K;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int row = (int)(i / K);
        int k = (int)(i - (int64_t)row * K);
        int c = k % p.C; int rs = k / p.C; int r = rs / p.S; int s = rs - r * p.S;
        if (p.flip) { r = p.R - 1 - r; s = p.S - 1 - s; }
        float v = w[row * p.s_row + c * p.s_c + r * p.s_r + s * p.s_s];
        float h = to_tf32_rn(v);
        hi[i] = h;
        lo[i] = v - h;
    }
}

// ---------------------------------------------------------------------------------------------
// fprop / dgrad kernel
// ---------------------------------------------------------------------------------------------
struct FwdParams {
    int M, N;                 // GEMM rows (output pixels n*P*Q) and columns (output channels)
    int P, Q;                 // output grid per image
    int kblocks, cblocks, S;  // K loop: taps * cblocks blocks of 32 channels; S = filter width
    int str_h, str_w, pad_h, pad_w, dil_h, dil_w;
    const float *bias, *mean, *inv_std, *gamma, *beta;
    int relu;
    float* out;               // [M][N]
};

template <int BN, int STAGES>
struct FwdSmem {
    static constexpr int A_BYTES = 128 * 128;   // 128 pixels x 32 floats
    static constexpr int B_BYTES = BN * 128;
    static constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
    static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
    static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;   // + barriers/flags + alignment slack
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(192, 1)
conv_tc_fwd_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_bhi,
                   const __grid_constant__ CUtensorMap tmap_blo, FwdParams p)
{
    using L = FwdSmem<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full_bar = (uint64_t*)(smem + L::BAR_OFFSET);
    uint64_t* xform_bar = full_bar + STAGES;
    uint64_t* empty_bar = xform_bar + STAGES;
    uint64_t* accum_bar = empty_bar + STAGES;
    uint32_t* tmem_slot = (uint32_t*)(accum_bar + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * 128, n0 = blockIdx.y * BN;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(&full_bar[s], 1); mbar_init(&xform_bar[s], 4); mbar_init(&empty_bar[s], 1); }
        mbar_init(accum_bar, 1);
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) { tmem_alloc(tmem_slot, BN); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            const int img = m0 / (p.P * p.Q);
            const int rem = m0 - img * (p.P * p.Q);
            const int p0 = rem / p.Q, q0 = rem - p0 * p.Q;
            const int base_w = q0 * p.str_w - p.pad_w, base_h = p0 * p.str_h - p.pad_h;
            for (int kb = 0; kb < p.kblocks; kb++) {
                const int s = kb % STAGES, use = kb / STAGES;
                if (use > 0 && !mbar_wait(&empty_bar[s], (use - 1) & 1, abort_flag, &g_tc_status, TC_ERR_EMPTY)) break;
                uint8_t* st = smem + s * L::STAGE_BYTES;
                const int tap = kb / p.cblocks, cb = kb - tap * p.cblocks;
                const int r = tap / p.S, sx = tap - r * p.S;
                mbar_expect_tx(&full_bar[s], L::A_BYTES + 2 * L::B_BYTES);
                tma_load_im2col_4d(st, &tmap_a, &full_bar[s], cb * 32, base_w, base_h, img,
                                   (uint16_t)(sx * p.dil_w), (uint16_t)(r * p.dil_h));
                tma_load_2d(st + 2 * L::A_BYTES, &tmap_bhi, &full_bar[s], kb * 32, n0);
                tma_load_2d(st + 2 * L::A_BYTES + L::B_BYTES, &tmap_blo, &full_bar[s], kb * 32, n0);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_tf32(128, BN, 0, 0);
            bool ok = true;
            for (int kb = 0; kb < p.kblocks && ok; kb++) {
                const int s = kb % STAGES, use = kb / STAGES;
                ok = mbar_wait(&full_bar[s], use & 1, abort_flag, &g_tc_status, TC_ERR_FULL) &&
                     mbar_wait(&xform_bar[s], use & 1, abort_flag, &g_tc_status, TC_ERR_XFORM);
                if (!ok) break;
                tc_fence_after();
                const uint32_t sa = smem_u32(smem + s * L::STAGE_BYTES);
                const uint64_t a_hi = make_smem_desc(sa, 0, 1024);
                const uint64_t a_lo = make_smem_desc(sa + L::A_BYTES, 0, 1024);
                const uint64_t b_hi = make_smem_desc(sa + 2 * L::A_BYTES, 0, 1024);
                const uint64_t b_lo = make_smem_desc(sa + 2 * L::A_BYTES + L::B_BYTES, 0, 1024);
#pragma unroll
                for (int k = 0; k < 4; k++) {           // 4 x (K = 8 tf32 = 32 bytes) per 128-byte row
                    const uint64_t adv = (uint64_t)(k * 2);
                    umma_tf32(tmem_base, a_lo + adv, b_hi + adv, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_tf32(tmem_base, a_hi + adv, b_lo + adv, idesc, 1u);
                    umma_tf32(tmem_base, a_hi + adv, b_hi + adv, idesc, 1u);
                }
                umma_commit(&empty_bar[s]);
            }
            if (ok) umma_commit(accum_bar);
        }
    } else {
        // ---------------- operand transform, then epilogue ----------------
        const int t = threadIdx.x - 64;      // 0..127
        bool ok = true;
        for (int kb = 0; kb < p.kblocks; kb++) {
            const int s = kb % STAGES, use = kb / STAGES;
            ok = mbar_wait(&full_bar[s], use & 1, abort_flag, &g_tc_status, TC_ERR_FULL);
            if (!ok) break;
            float4* a_hi = (float4*)(smem + s * L::STAGE_BYTES);
            float4* a_lo = (float4*)(smem + s * L::STAGE_BYTES + L::A_BYTES);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                float4 v = a_hi[t + i * 128];
                float4 h, l;
                h.x = to_tf32_rn(v.x); h.y = to_tf32_rn(v.y); h.z = to_tf32_rn(v.z); h.w = to_tf32_rn(v.w);
                l.x = v.x - h.x; l.y = v.y - h.y; l.z = v.z - h.z; l.w = v.w - h.w;
                a_hi[t + i * 128] = h;
                a_lo[t + i * 128] = l;
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&xform_bar[s]);
        }
        if (ok) ok = mbar_wait(accum_bar, 0, abort_flag, &g_tc_status, TC_ERR_ACCUM);
        if (ok) {
            tc_fence_after();
            const int quad = warp & 3;                       // TMEM lane quadrant this warp may read
            const int m = m0 + quad * 32 + lane;
            float* orow = p.out + (int64_t)m * p.N;
#pragma unroll 1
            for (int c = 0; c < BN / 32; c++) {
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(c * 32), r);
                tmem_ld_wait();
                if (m < p.M) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const int n = n0 + c * 32 + j;
                        if (n >= p.N) break;
                        float v[4];
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            float a = __uint_as_float(r[j + e]);
                            const int ne = n + e;
                            if (p.bias) a += p.bias[ne];
                            if (p.mean) { float tt = (a - p.mean[ne]) * p.inv_std[ne]; a = tt * p.gamma[ne] + p.beta[ne]; }
                            if (p.relu) a = fmaxf(a, 0.f);
                            v[e] = a;
                        }
                        *reinterpret_cast<float4*>(orow + n) = make_float4(v[0], v[1], v[2], v[3]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, BN); }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const int*, const int*, cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode_tiled = nullptr;
static EncodeIm2colFn g_encode_im2col = nullptr;

static bool load_driver_entry_points()
{
    if (g_encode_tiled && g_encode_im2col) return true;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) return false;
    g_encode_tiled = (EncodeTiledFn)fn;
    fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) return false;
    g_encode_im2col = (EncodeIm2colFn)fn;
    return true;
}

// 2-D row-major float matrix [rows][cols], box = 32 columns x box_rows rows, 128B swizzle.
static bool make_map_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows)
{
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * sizeof(float)};
    cuuint32_t box[2] = {32, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return g_encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// NHWC activation tensor (n, h, w, c) seen through an im2col window: `pixels` consecutive output
// pixels x 32 channels per load. Corners are given in (w, h) order.
static bool make_map_im2col(CUtensorMap* map, const void* base, int n, int h, int w, int c, int pad_h, int pad_w,
                            int kh, int kw, int dil_h, int dil_w, int str_h, int str_w, uint32_t pixels)
{
    cuuint64_t dims[4] = {(cuuint64_t)c, (cuuint64_t)w, (cuuint64_t)h, (cuuint64_t)n};
    cuuint64_t strides[3] = {(cuuint64_t)c * 4, (cuuint64_t)w * c * 4, (cuuint64_t)h * w * c * 4};
    int lower[2] = {-pad_w, -pad_h};
    int upper[2] = {pad_w - (kw - 1) * dil_w, pad_h - (kh - 1) * dil_h};
    cuuint32_t estr[4] = {1, (cuuint32_t)str_w, (cuuint32_t)str_h, 1};
    return g_encode_im2col(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(base), dims, strides, lower, upper,
                           32, pixels, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static bool corners_ok(int v) { return v >= -128 && v <= 127; }

bool tc_supported(const Geo& g, int pass)
{
    if (g.dtype != B2C_F32 || g.layout != B2C_LAYOUT_NHWC || g.engine == B2C_ENGINE_FMA) return false;
    if (g.vstr > 8 || g.hstr > 8) return false;
    if ((g.kh - 1) * g.vdil > 255 || (g.kw - 1) * g.hdil > 255) return false;
    if (pass == B2C_PASS_FPROP) {
        if (g.ci % 32 || g.co % 4) return false;
        return corners_ok(-g.vpad) && corners_ok(-g.hpad) && corners_ok(g.vpad - (g.kh - 1) * g.vdil) &&
               corners_ok(g.hpad - (g.kw - 1) * g.hdil);
    }
    if (pass == B2C_PASS_DGRAD) {
        if (g.vstr != 1 || g.hstr != 1) return false;
        if (g.co % 32 || g.ci % 4) return false;
        int pv = (g.kh - 1) * g.vdil - g.vpad, ph = (g.kw - 1) * g.hdil - g.hpad;
        if (pv < 0 || ph < 0) return false;
        return corners_ok(-pv) && corners_ok(-ph) && corners_ok(pv - (g.kh - 1) * g.vdil) && corners_ok(ph - (g.kw - 1) * g.hdil);
    }
    return false;
}

static size_t fwd_filter_bytes(const Geo& g, int pass)
{
    int rows = pass == B2C_PASS_FPROP ? g.co : g.ci;
    int C = pass == B2C_PASS_FPROP ? g.ci : g.co;
    return align_up((size_t)rows * g.kh * g.kw * C * sizeof(float), 1024);
}

size_t tc_workspace_bytes(const Geo& g, int pass)
{
    if (pass == B2C_PASS_FPROP || pass == B2C_PASS_DGRAD) return 2 * fwd_filter_bytes(g, pass) + 1024;
    return 0;
}

template <int BN, int STAGES>
static int launch_fwd(const CUtensorMap& ma, const CUtensorMap& mbh, const CUtensorMap& mbl, const FwdParams& p, cudaStream_t st)
{
    using L = FwdSmem<BN, STAGES>;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(conv_tc_fwd_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) { set_cuda_error(e, "cudaFuncSetAttribute(conv_tc_fwd_kernel)"); return B2C_ERR_CUDA; }
        attr_set = true;
    }
    dim3 grid((p.M + 127) / 128, (p.N + BN - 1) / BN);
    if (grid.y > 65535) return B2C_ERR_TOO_LARGE;
    conv_tc_fwd_kernel<BN, STAGES><<<grid, 192, L::TOTAL, st>>>(ma, mbh, mbl, p);
    return check_launch("conv_tc_fwd_kernel");
}

// Shared by fprop and dgrad: `act` is the gathered NHWC tensor (n, ah, aw, C), the filter source is
// described by PrepParams, the output is [n*P*Q][N].
static int run_fwd(int n, int ah, int aw, int C, int P, int Q, int N, int kh, int kw, int pad_h, int pad_w, int str_h,
                   int str_w, int dil_h, int dil_w, const void* act, const void* w, const PrepParams& pp,
                   const void* bias, const b2c_bn_params* bn, int relu, void* out, void* ws, size_t ws_bytes,
                   cudaStream_t st)
{
    if (!load_driver_entry_points()) return B2C_ERR_UNSUPPORTED;
    const int64_t K = (int64_t)kh * kw * C;
    const size_t fbytes = align_up((size_t)N * K * sizeof(float), 1024);
    uintptr_t base = align_up((uintptr_t)ws, 1024);
    if (!ws || base + 2 * fbytes > (uintptr_t)ws + ws_bytes) return B2C_ERR_WORKSPACE_TOO_SMALL;
    if (((uintptr_t)act & 15) || ((uintptr_t)out & 15)) return B2C_ERR_MISALIGNED;
    float* w_hi = (float*)base;
    float* w_lo = (float*)(base + fbytes);
    {
        int64_t total = (int64_t)N * K;
        int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
        tc_prep_filter_kernel<<<blocks, 256, 0, st>>>(pp, (const float*)w, w_hi, w_lo);
        int rc = check_launch("tc_prep_filter_kernel");
        if (rc) return rc;
    }
    const int BN = N <= 64 ? 64 : 128;
    CUtensorMap ma, mbh, mbl;
    if (!make_map_im2col(&ma, act, n, ah, aw, C, pad_h, pad_w, kh, kw, dil_h, dil_w, str_h, str_w, 128)) return B2C_ERR_UNSUPPORTED;
    if (!make_map_2d(&mbh, w_hi, N, K, BN) || !make_map_2d(&mbl, w_lo, N, K, BN)) return B2C_ERR_UNSUPPORTED;
    FwdParams p{};
    p.M = n * P * Q; p.N = N; p.P = P; p.Q = Q;
    p.cblocks = C / 32; p.kblocks = kh * kw * p.cblocks; p.S = kw;
    p.str_h = str_h; p.str_w = str_w; p.pad_h = pad_h; p.pad_w = pad_w; p.dil_h = dil_h; p.dil_w = dil_w;
    p.bias = (const float*)bias;
    if (bn) { p.mean = (const float*)bn->mean; p.inv_std = (const float*)bn->inv_std; p.gamma = (const float*)bn->gamma; p.beta = (const float*)bn->beta; }
    p.relu = relu;
    p.out = (float*)out;
    if (BN == 64) return launch_fwd<64, 4>(ma, mbh, mbl, p, st);
    return launch_fwd<128, 3>(ma, mbh, mbl, p, st);
}

int tc_fprop(const Geo& g, const void* x, const void* w, const void* bias, const b2c_bn_params* bn, int relu,
             void* y, void* ws, size_t ws_bytes, cudaStream_t st)
{
    WStride wsd = w_stride(g.w_layout, g.ci, g.co, g.kh, g.kw);
    PrepParams pp{g.co, g.ci, g.kh, g.kw, wsd.sk, wsd.sc, wsd.sr, wsd.ss, 0};
    return run_fwd(g.n, g.h, g.w, g.ci, g.ho, g.wo, g.co, g.kh, g.kw, g.vpad, g.hpad, g.vstr, g.hstr, g.vdil, g.hdil,
                   x, w, pp, bias, bn, relu, y, ws, ws_bytes, st);
}

int tc_dgrad(const Geo& g, const void* dy, const void* w, void* dx, void* ws, size_t ws_bytes, cudaStream_t st)
{
    WStride wsd = w_stride(g.w_layout, g.ci, g.co, g.kh, g.kw);
    // rows = ci, gathered channels = co, taps flipped
    PrepParams pp{g.ci, g.co, g.kh, g.kw, wsd.sc, wsd.sk, wsd.sr, wsd.ss, 1};
    const int pv = (g.kh - 1) * g.vdil - g.vpad, ph = (g.kw - 1) * g.hdil - g.hpad;
    return run_fwd(g.n, g.ho, g.wo, g.co, g.h, g.w, g.ci, g.kh, g.kw, pv, ph, 1, 1, g.vdil, g.hdil,
                   dy, w, pp, nullptr, nullptr, 0, dx, ws, ws_bytes, st);
}

int tc_wgrad(const Geo&, const void*, const void*, void*, void*, void*, size_t, cudaStream_t) { return B2C_ERR_UNSUPPORTED; }

int tc_read_status(int* out)
{
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int));
    if (e != cudaSuccess) { set_cuda_error(e, "cudaMemcpyFromSymbol(g_tc_status)"); return B2C_ERR_CUDA; }
    if (v != 0) { int zero = 0; cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int)); }
    *out = v;
    return B2C_OK;
}

}  // namespace b2c

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
//           -- the same kernel run on dy with padding (k-1)*dil - pad; the flipped tap is a TMA coordinate
//              into the caller's filter, not a copy
//   wgrad : dw[co][tap][ci] = sum_pixel x[pixel+tap][ci] * dy[pixel][co]           (split over pixels)
//
// 3xTF32: every float32 operand a is split as a = hi + lo with hi = a with the low 13 mantissa bits
// cleared (what the tensor core reads of a float32 anyway) and lo = a - hi (exact in float32).  Three
// tensor-core products lo*hi + hi*lo + hi*hi accumulate in the float32 TMEM tile (small terms first).
// The A tile (activations; x^T in wgrad) is split by the transform warps, which read it once from shared
// memory and write hi and lo into tensor memory with tcgen05.st; the MMAs take A from tensor memory and only B
// from shared memory.  The B tile (filters; dy in wgrad) is loaded by TMA straight from the caller's tensor and
// its lo half is written in shared memory by the same warps; long launches and filter layouts without a
// contiguous channel axis use hi/lo copies written once per call by a small kernel instead.
//
// Variants (template parameters): whole tiles or balanced (tile, k-block) ranges with a hand-over of partial
// tiles between consecutive CTAs; the filter from split copies or read in place (K-major or MN-major); a chunked
// drain, or for tiles of one chunk a streaming epilogue (32 columns at a time straight from tensor memory) with four
// or eight drain warps; for tiles of at most four k-blocks the filter tiles of the CTA's column tile resident in
// shared memory for the whole launch; several pixel classes (a strided data gradient) in one launch.  NCHW tensors
// run on channel-last copies.
//
// Warp roles (320 threads; 448 with eight drain warps): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer
// (both stay converged and issue through one elected lane), warps 2-5 = operand transform,
// warps 6-9 (6-13) = drain + epilogue: the tensor core's accumulate step truncates, so sums are kept in
// tensor memory only for a chunk of 8 k-blocks (two TMEM buffers alternate) and added chunk by
// chunk into float32 registers with round-to-nearest, then bias / BN-scale / ReLU -> global.
// Every mbarrier wait is bounded: when a wait runs out the CTA raises an abort flag, records a
// status word in global memory, skips its remaining work, frees its tensor memory and returns.
#include "b2c_common.cuh"
#include <cuda.h>
#include <stdlib.h>
#include <mutex>

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

// One lane of the (converged) warp is chosen; the compiler knows that exactly one thread runs the guarded
// code, which lets it keep descriptors, coordinates and barrier addresses in uniform registers, the form
// the TMA and tensor-core instructions take their operands in.
__device__ __forceinline__ bool elect_one_sync() {
    uint32_t pred = 0;
    asm volatile("{\n\t.reg .b32 rx;\n\t.reg .pred px;\n\telect.sync rx|px, %1;\n\tselp.u32 %0, 1, 0, px;\n\t}"
                 : "=r"(pred) : "r"(0xFFFFFFFFu));
    return pred != 0;
}

#define TC_WAIT_CYCLES 2000000000LL   // about one second at the boost clock

// Bounded wait. Returns false when the wait ran out or another role already gave up.
// mbarrier.try_wait suspends the thread in hardware for a short while, so the loop is not hot; the abort
// flag and the clock are looked at only every 32 failed tries to keep waiting warps off the LSU and the
// issue ports the working warps need.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int code,
                                          long long limit_cycles = TC_WAIT_CYCLES) {
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = 0;
    uint32_t tries = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++tries & 31u) == 0) {
            if (*abort_flag) return false;
            const long long now = clock64();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit_cycles) {
                *abort_flag = 1;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}

__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Start fetching a tensor map (a kernel parameter) into the TMA unit's descriptor cache.
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tma_load_im2col_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c, int w, int h,
                                                   int n, uint16_t off_w, uint16_t off_h) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes"
                 " [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h)
                 : "memory");
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(smem_u32(src)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* src, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(map), "r"(smem_u32(src)), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Wait until at most N of this thread's committed store groups still read their shared-memory source.
template <int N> __device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }

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
// D[tmem] (+)= A[tmem] * B[smem]: the A tile sits in tensor memory (row m in lane m, one tf32 element per
// 32-bit column, K-major), so only B is fetched from shared memory.
__device__ __forceinline__ void umma_tf32_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
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
// The same load with the 32 columns landing in float registers r[0..31] (constant indices after inlining).
__device__ __forceinline__ void tmem_ld_32x32_f(uint32_t taddr, float* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]),
                   "=f"(r[8]), "=f"(r[9]), "=f"(r[10]), "=f"(r[11]), "=f"(r[12]), "=f"(r[13]), "=f"(r[14]), "=f"(r[15]),
                   "=f"(r[16]), "=f"(r[17]), "=f"(r[18]), "=f"(r[19]), "=f"(r[20]), "=f"(r[21]), "=f"(r[22]), "=f"(r[23]),
                   "=f"(r[24]), "=f"(r[25]), "=f"(r[26]), "=f"(r[27]), "=f"(r[28]), "=f"(r[29]), "=f"(r[30]), "=f"(r[31])
                 : "r"(taddr) : "memory");
}
// Registers -> tensor memory: lane i of the warp writes r[0..31] to columns taddr.col .. +31 of TMEM lane
// (taddr.lane + i); a warp may only touch the 32-lane quadrant (warp index mod 4).
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                 "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float to_tf32_rn(float v) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return __uint_as_float(r);
}

// Shared-memory matrix descriptor for tiles made of 128-byte rows.
//  K-major (layout 2 = 128B swizzle): a row is 32 K elements of one M/N row; 8-row groups lie
//    `sbo_bytes` (1024) apart; the leading offset is unused.
//  MN-major (layout 1 = 128B swizzle with 32-byte atoms, the only MN-major layout tf32 operands may
//    use): a row is 32 M/N elements of one K index; 4-row K groups lie `sbo_bytes` (512) apart and
//    further 32-element M/N groups `lbo_bytes` apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;     // descriptor version for sm_100
    d |= (uint64_t)layout << 61;
    return d;
}
// Instruction descriptor: tf32 x tf32 -> f32, dense.
__host__ __device__ constexpr uint32_t make_idesc_tf32(int M, int N, int a_mn_major, int b_mn_major) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// Device status word shared by all tensor-core kernels (0 = fine).
__device__ int g_tc_status = 0;

// Hand-over flags of the balanced mode (4 per CTA).  They live in the library image, start as zeros and are returned
// to zero by the warp that consumes them, so no launch has to clear them first.  A bank belongs to one stream
// (kernels of one stream never overlap); a stream beyond the bank count gets its flags in the caller's workspace,
// cleared before the launch.
#define TC_SYNC_BANKS 8
#define TC_SYNC_WORDS 4096
#define TC_SYNC_FLAGS 4096
static __device__ __align__(256) unsigned int g_tc_sync[TC_SYNC_BANKS * TC_SYNC_WORDS];

enum { TC_ERR_FULL = 1, TC_ERR_XFORM = 2, TC_ERR_EMPTY = 3, TC_ERR_TFULL = 4, TC_ERR_TEMPTY = 5, TC_ERR_PARTIAL = 6, TC_ERR_SELFTEST = 7 };

#if defined(B2C_TC_PROFILE) || defined(B2C_TC_SWITCHES)
#define B2C_TC_DEV 1
#endif
#ifdef B2C_TC_PROFILE
// Development build only: per-role cycle counters of CTA 0 (slots documented at the call sites).
__device__ long long g_tc_prof[32];
#define TC_PROF_DECL() long long _pa[16]; for (int _i = 0; _i < 16; _i++) _pa[_i] = 0
#define TC_PROF_T0() long long _pt = clock64()
#define TC_PROF_RESET() _pt = clock64()
#define TC_PROF_ADD(slot) do { long long _n = clock64(); _pa[slot] += _n - _pt; _pt = _n; } while (0)
#define TC_PROF_FLUSH() do { if (blockIdx.x == 0) for (int _i = 0; _i < 16; _i++) if (_pa[_i]) atomicAdd((unsigned long long*)&g_tc_prof[_i], (unsigned long long)_pa[_i]); } while (0)
#else
#define TC_PROF_DECL() do { } while (0)
#define TC_PROF_T0() do { } while (0)
#define TC_PROF_RESET() do { } while (0)
#define TC_PROF_ADD(slot) do { } while (0)
#define TC_PROF_FLUSH() do { } while (0)
#endif

// ---------------------------------------------------------------------------------------------
// Filter preparation: hi/lo split into the K-major GEMM layout the fprop/dgrad kernel reads by TMA
// ---------------------------------------------------------------------------------------------
struct PrepParams {
    int rows, C, R, S;               // output is [rows][(r*S+s)*C + c], r < R, s < S (virtual taps)
    int64_t s_row, s_c, s_r, s_s;    // element strides of the source filter by (row, c, r, s)
    int r0, rstep, s0, sstep;        // real tap of virtual tap (r, s): (r0 + rstep*r, s0 + sstep*s)
    int Rreal, Sreal;                // extent of the real filter
};

// Also clears `nflags` ints at `flags` (the hand-over flags of the balanced mode of the convolution kernel that
// follows in the stream), which saves a separate memset.
__global__ void tc_prep_filter_kernel(PrepParams p, const float* __restrict__ w, float* __restrict__ hi, float* __restrict__ lo,
                                      int* __restrict__ flags, int nflags)
{
    pdl_prologue();
    if (blockIdx.x == 0) for (int i = threadIdx.x; i < nflags; i += blockDim.x) flags[i] = 0;
    int64_t K = (int64_t)p.R * p.S * p.C;
    int64_t total = (int64_t)p.rows * K;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int row = (int)(i / K);
        int k = (int)(i - (int64_t)row * K);
        int c = k % p.C; int rs = k / p.C; int r = rs / p.S; int s = rs - r * p.S;
        r = p.r0 + p.rstep * r; s = p.s0 + p.sstep * s;
        float v = w[row * p.s_row + c * p.s_c + r * p.s_r + s * p.s_s];
        float h = to_tf32_rn(v);
        hi[i] = h;
        lo[i] = v - h;
    }
}

// ---------------------------------------------------------------------------------------------
// Few-channel layers (the Ci=3 network stem): the TMA gather needs 32-channel, 16-byte aligned rows, so
// for these the im2row matrix is written out once, [pixel][(r*S+s)*C + c] zero-padded to a multiple of
// 32 columns, and the layer then runs as a 1x1 convolution over it.  With C*R*S small the matrix costs
// less HBM traffic than the output tensor it produces.
// ---------------------------------------------------------------------------------------------
struct LowerParams { int n, h, w, c, ho, wo, kh, kw, vpad, hpad, vstr, hstr, vdil, hdil, K, Kp; };

// The grid's thread count is a multiple of the float4 count of a row (Kp / 4), so a thread keeps its column
// group for the whole grid-stride loop: the four (tap, channel) pairs are decoded once into registers and the
// pixel advances by a constant step, carried through (w, h, n) without divisions.
__global__ void tc_lower_kernel(LowerParams p, const float* __restrict__ x, float4* __restrict__ rows)
{
    pdl_prologue();
    const int kq = p.Kp / 4;
    const int64_t total = (int64_t)p.n * p.ho * p.wo * kq;
    const int64_t threads = (int64_t)gridDim.x * blockDim.x;          // multiple of kq (see launch_lower)
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int q4 = (int)(i % kq);
    int dh[4], dwc[4], off[4];
#pragma unroll
    for (int e = 0; e < 4; e++) {
        const int k = q4 * 4 + e;
        if (k < p.K) {
            const int c = k % p.c, rs = k / p.c, r = rs / p.kw, sx = rs - r * p.kw;
            dh[e] = r * p.vdil; dwc[e] = sx * p.hdil; off[e] = (dh[e] * p.w + dwc[e]) * p.c + c;
        } else { dh[e] = 1 << 28; dwc[e] = 0; off[e] = 0; }          // padding column: always out of range
    }
    int64_t m = i / kq;
    int ow = (int)(m % p.wo); m /= p.wo;
    int oh = (int)(m % p.ho); int nn = (int)(m / p.ho);
    int64_t step = threads / kq;                                     // pixels per grid stride
    const int s_w = (int)(step % p.wo); step /= p.wo;
    const int s_h = (int)(step % p.ho); const int s_n = (int)(step / p.ho);
    for (; i < total; i += threads) {
        const int h0 = oh * p.vstr - p.vpad, w0 = ow * p.hstr - p.hpad;
        const float* base = x + (((int64_t)nn * p.h + h0) * p.w + w0) * p.c;
        float v[4];
#pragma unroll
        for (int e = 0; e < 4; e++)
            v[e] = ((unsigned)(h0 + dh[e]) < (unsigned)p.h && (unsigned)(w0 + dwc[e]) < (unsigned)p.w) ? __ldg(base + off[e]) : 0.f;
        rows[i] = make_float4(v[0], v[1], v[2], v[3]);
        ow += s_w; if (ow >= p.wo) { ow -= p.wo; oh++; }
        oh += s_h; if (oh >= p.ho) { oh -= p.ho; nn++; }
        nn += s_n;
    }
}

// The same matrix, one block per output row (n, oh): the kh input rows the row of windows touches are copied into
// shared memory once (coalesced, zero outside the image), then every float4 of the matrix row block is put
// together from four shared-memory reads.  Threads are laid out as (pixel sub-index, column group), so a thread
// again keeps its column group and decodes its four (tap, channel) pairs once.
__global__ void tc_lower_rows_kernel(LowerParams p, const float* __restrict__ x, float4* __restrict__ rows, int wp)
{
    pdl_prologue();
    extern __shared__ float patch[];                      // [kh][wp][c], column j is input column j - hpad
    const int nn = blockIdx.x / p.ho, oh = blockIdx.x - nn * p.ho;
    const int rowlen = wp * p.c;
    // one patch pixel per thread and trip (its few channels in an inner loop: no division per element)
    for (int r = 0; r < p.kh; r++) {
        const int ih = oh * p.vstr - p.vpad + r * p.vdil;
        const bool row_in = (unsigned)ih < (unsigned)p.h;
        const float* src = x + ((int64_t)nn * p.h + ih) * p.w * p.c;
        for (int j = threadIdx.x; j < wp; j += blockDim.x) {
            const int iw = j - p.hpad;
            const bool in = row_in && (unsigned)iw < (unsigned)p.w;
            float* dst = patch + r * rowlen + j * p.c;
            for (int c = 0; c < p.c; c++) dst[c] = in ? __ldg(src + (int64_t)iw * p.c + c) : 0.f;
        }
    }
    __syncthreads();
    const int kq = p.Kp / 4;
    const int sub = threadIdx.x / kq, q4 = threadIdx.x - sub * kq, nsub = blockDim.x / kq;
    if (sub >= nsub) return;
    int off[4];
    bool real[4];
#pragma unroll
    for (int e = 0; e < 4; e++) {
        const int k = q4 * 4 + e;
        real[e] = k < p.K;
        const int kk = real[e] ? k : 0;
        const int c = kk % p.c, rs = kk / p.c, r = rs / p.kw, sx = rs - r * p.kw;
        off[e] = r * rowlen + sx * p.hdil * p.c + c;
    }
    float4* dst = rows + ((int64_t)nn * p.ho + oh) * p.wo * kq + q4;
    for (int ow = sub; ow < p.wo; ow += nsub) {
        const float* base = patch + ow * p.hstr * p.c;
        float4 v;
        v.x = real[0] ? base[off[0]] : 0.f; v.y = real[1] ? base[off[1]] : 0.f;
        v.z = real[2] ? base[off[2]] : 0.f; v.w = real[3] ? base[off[3]] : 0.f;
        dst[(int64_t)ow * kq] = v;
    }
}

// hi/lo split of the filter in the lowered column order, zero in the padding columns
__global__ void tc_prep_filter_lowered_kernel(int rows, int K, int Kp, int C, int S, int64_t s_row, int64_t s_c, int64_t s_r,
                                              int64_t s_s, const float* __restrict__ w, float* __restrict__ hi, float* __restrict__ lo)
{
    pdl_prologue();
    const int64_t total = (int64_t)rows * Kp;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int row = (int)(i / Kp), k = (int)(i - (int64_t)row * Kp);
        float v = 0.f;
        if (k < K) { const int c = k % C, rs = k / C, r = rs / S, sx = rs - r * S; v = w[row * s_row + c * s_c + r * s_r + sx * s_s]; }
        const float h = to_tf32_rn(v);
        hi[i] = h; lo[i] = v - h;
    }
}

// ---------------------------------------------------------------------------------------------
// The kernel (one template, two modes)
// ---------------------------------------------------------------------------------------------
enum { TCM_FWD = 0, TCM_WGRAD = 1 };
// Where the FWD kernel takes its B tiles (filters) from:
//  TCB_SPLIT  hi and lo copies in the K-major GEMM layout, written by tc_prep_filter_kernel (any filter layout)
//  TCB_RAW_K  the caller's filter itself, read through a 3-D tensor map (channel, tap, row) whose channel axis is
//             the GEMM K axis: K-major tiles; the transform warps write the lo half in shared memory
//  TCB_RAW_MN the same with the channel axis being the GEMM N axis: MN-major boxes as in WGRAD
enum { TCB_SPLIT = 0, TCB_RAW_K = 1, TCB_RAW_MN = 2 };

#define TC_CHUNK 8   // k-blocks accumulated in tensor memory before the partial sum is drained

struct TcParams {
    // FWD: GEMM rows = output pixels, columns = output channels. WGRAD: rows = (tap, ci), columns = co.
    int M, N;
    int P, Q;                  // pixel grid per image the pixel index runs over
    int kblocks;               // FWD: taps * cblocks.  WGRAD: 32-pixel blocks per split
    int cblocks, S;            // channel blocks of 32 per tap, filter width
    int C;                     // gathered channels per tap
    int str_h, str_w, dil_h, dil_w;
    int low_h, low_w;          // lower corner of the im2col window (= -padding for a plain convolution)
    int Mpix;                  // WGRAD: total pixels
    int a_box_log2;            // WGRAD: log2 of the channels per x box (32, 64 or 128: the widest that divides C)
    int splits;                // WGRAD: pixel ranges (1 for FWD)
    // FWD epilogue
    const float *bias, *mean, *inv_std, *gamma, *beta;
    int relu;
    float* out;                // FWD: row m=(n,i,j) at out + n*o_sn + i*o_sh + j*o_sw.  WGRAD: partial [split][M][N]
    int64_t o_sn, o_sh, o_sw;
    int epi;                   // TC_EPI_* bits: which per-channel steps the FWD epilogue applies
#ifdef B2C_TC_DEV
    int dbg;                   // development build only: 2 = issue one MMA of three, 4 = transform warps do no work
#endif
    // Balanced mode (FWD only): the (tile, k-block) work units are cut into equal contiguous ranges, one per CTA,
    // so a tile may be shared by consecutive CTAs.  The CTA that starts a tile owns it; the others store their
    // partial tile in `sk_partial` (slot = CTA index, [BN/4][128 rows][4] floats) and raise `sk_flags` (4 per slot, one per
    // drain warp); the owner adds the partials in CTA order and runs the epilogue.
    int tap_r0, tap_rstep, tap_s0, tap_sstep, tap_sreal;   // raw-filter modes: real tap of virtual tap (r, s)
    int sk;
    float* sk_partial;
    int* sk_flags;
    float* db_partial;         // WGRAD: per-(split, transform warp) channel sums of dy, [splits][4][N], or null
    int tma_store;             // output rows are dense [M][N] (or [split][M][N]): store tiles through the output tensor map
    int sk_selfclean;          // balanced mode: the owner returns a consumed flag to zero (flags in the library's bank)
    // FWD writing one parity class of a stride-2 data gradient whose other three classes are zeros (a 1x1 filter): with
    // zfill set, every output row also stores zeros at the pixel to its right, below it and diagonally below (offsets
    // z_w, z_h, z_w + z_h elements) where those pixels exist (2 q + 1 < z_W, 2 p + 1 < z_H), so dx needs no clearing pass.
    int zfill, z_W, z_H;
    int64_t z_w, z_h;
    // FWD over several pixel classes in one launch (the parity classes of a strided data gradient): the tile list is
    // the concatenation of the classes' tile lists, class c owning tiles [cls_tile0[c], cls_tile0[c + 1]).  A class has
    // its own pixel grid, window corner, tap set, k-block count, output offset and activation tensor map; channel
    // counts, filter and output strides are the launch's.  Used by the MULTI variants only.
    int ncls;
    int cls_tile0[5];
    int cls_M[4], cls_P[4], cls_Q[4], cls_kblocks[4], cls_S[4], cls_low_h[4], cls_low_w[4], cls_r0[4], cls_s0[4];
    int64_t cls_out[4];
    // FWD with batch statistics: for every block of 32 output rows, row (m / 32) of `stats` ([ceil(M/32)][2][N] floats)
    // receives the per-channel sum and sum of squares of the stored values (rows past M left out).  Null: off.
    // stats_cta: the grid is a multiple of the column-tile count nt, so a CTA keeps one column tile; it adds the sums
    // of all its tiles in registers and `stats` is [(grid / nt) * 4][2][N]: one row per CTA group and row quadrant.
    float* stats;
    int stats_cta;
};

// Per-channel epilogue steps of the forward pass, decided once on the host so the drain warps branch on
// one register instead of testing three pointers per element.
enum { TC_EPI_BIAS = 1, TC_EPI_BN = 2, TC_EPI_RELU = 4, TC_EPI_VEC = 8 };

// bias / BN-scale / ReLU on the 32 accumulators a[0..31] of one output row, channels nbase..nbase+31.
// The per-channel vectors are read at warp-uniform addresses (every lane owns a different row of the
// same channels); with TC_EPI_VEC (all vectors 16-byte aligned, N a multiple of 4) four channels per load.
__device__ __forceinline__ void tc_epilogue_math(const TcParams& p, int nbase, float* a)
{
    if (p.epi & TC_EPI_VEC) {
        if (p.epi & TC_EPI_BIAS) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
                if (nbase + j < p.N) {
                    const float4 b = __ldg(reinterpret_cast<const float4*>(p.bias + nbase + j));
                    a[j] += b.x; a[j + 1] += b.y; a[j + 2] += b.z; a[j + 3] += b.w;
                }
        }
        if (p.epi & TC_EPI_BN) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
                if (nbase + j < p.N) {
                    const float4 mu = __ldg(reinterpret_cast<const float4*>(p.mean + nbase + j));
                    const float4 is = __ldg(reinterpret_cast<const float4*>(p.inv_std + nbase + j));
                    const float4 ga = __ldg(reinterpret_cast<const float4*>(p.gamma + nbase + j));
                    const float4 be = __ldg(reinterpret_cast<const float4*>(p.beta + nbase + j));
                    float t;
                    t = (a[j] - mu.x) * is.x;     a[j] = t * ga.x + be.x;
                    t = (a[j + 1] - mu.y) * is.y; a[j + 1] = t * ga.y + be.y;
                    t = (a[j + 2] - mu.z) * is.z; a[j + 2] = t * ga.z + be.z;
                    t = (a[j + 3] - mu.w) * is.w; a[j + 3] = t * ga.w + be.w;
                }
        }
    } else {
        if (p.epi & TC_EPI_BIAS) {
#pragma unroll
            for (int j = 0; j < 32; j++)
                if (nbase + j < p.N) a[j] += __ldg(p.bias + nbase + j);
        }
        if (p.epi & TC_EPI_BN) {
#pragma unroll
            for (int j = 0; j < 32; j++)
                if (nbase + j < p.N) {
                    const float t = (a[j] - __ldg(p.mean + nbase + j)) * __ldg(p.inv_std + nbase + j);
                    a[j] = t * __ldg(p.gamma + nbase + j) + __ldg(p.beta + nbase + j);
                }
        }
    }
    if (p.epi & TC_EPI_RELU) {
#pragma unroll
        for (int j = 0; j < 32; j++) a[j] = fmaxf(a[j], 0.f);
    }
}

// Shared memory per pipeline stage: the raw A tile (activations), then the hi and lo halves of the B tile.
// Tensor memory (512 columns): two accumulator buffers of BN columns, then per stage 64 columns holding
// the hi and lo halves of the A tile (128 rows x 32 k).
// RESKB > 0 (resident filters): the B tiles of all k-blocks (at most RESKB) stay in shared memory for the whole launch,
// a stage holds the A tile only, and the A slots in tensor memory (TSLOTS of them) cycle separately from the STAGES
// shared-memory stages.
template <int BN, int STAGES, int SLABS, int DRAIN_WARPS = 4, int RESKB = 0>
struct TcSmem {
    static constexpr int A_BYTES = 128 * 128;   // 128 rows x 32 floats (FWD) or 32 pixels x 128 rows (WGRAD)
    static constexpr int B_BYTES = BN * 128;
    static constexpr int STAGE_BYTES = RESKB ? A_BYTES : A_BYTES + 2 * B_BYTES;
    static constexpr int RES_OFFSET = STAGES * STAGE_BYTES;         // resident B tiles: per k-block the raw tile, then its lo half
    static constexpr int BAR_OFFSET = RES_OFFSET + RESKB * 2 * B_BYTES;
    static constexpr int TSLOTS = RESKB ? (512 - 2 * BN) / 64 : STAGES;
    static constexpr int EPI_OFFSET = BAR_OFFSET + 1024;          // barriers and flags live in the first 512 bytes
    static constexpr int EPI_BYTES = DRAIN_WARPS * SLABS * 4096;  // per drain warp: SLABS 32 x 32 float staging slabs
    static constexpr int TOTAL = EPI_OFFSET + EPI_BYTES + 1024;   // + alignment slack
    static constexpr int TMEM_A_COL = 2 * BN;                     // first column of the A slots
    static constexpr int TMEM_COLS = 512;
    static_assert(2 * BN + TSLOTS * 64 <= TMEM_COLS, "tensor memory budget");
    static_assert(TOTAL <= 232448, "shared memory budget");
};

// The sequence of (tile, k-block range) segments one CTA works through; every warp role walks the same sequence.
// Plain mode: whole tiles blockIdx.x, blockIdx.x + gridDim.x, ...  Balanced mode: the contiguous unit range
// [total * b / G, total * (b + 1) / G) of CTA b, unit = tile * kblocks + kb.
struct TileWalk {
    int tile, kb_b, kb_e;
    int next_tile, total_tiles, kblocks;
    long long u, u_end;
    __device__ __forceinline__ static long long range_begin(long long total, int cta, int ctas) { return total * cta / ctas; }
    __device__ __forceinline__ void init(int total_tiles_, int kblocks_) {
        total_tiles = total_tiles_; kblocks = kblocks_; next_tile = blockIdx.x;
        const long long total = (long long)total_tiles_ * kblocks_;
        u = range_begin(total, blockIdx.x, gridDim.x); u_end = range_begin(total, blockIdx.x + 1, gridDim.x);
    }
    template <bool BALANCED> __device__ __forceinline__ bool next() {
        if (!BALANCED) {
            if (next_tile >= total_tiles) return false;
            tile = next_tile; next_tile += gridDim.x; kb_b = 0; kb_e = kblocks;
            return true;
        }
        if (u >= u_end) return false;
        tile = (int)(u / kblocks);
        kb_b = (int)(u - (long long)tile * kblocks);
        const long long rem = u_end - u;
        kb_e = (long long)kb_b + rem < (long long)kblocks ? kb_b + (int)rem : kblocks;
        u += kb_e - kb_b;
        return true;
    }
};

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Registers are handed out per group of four warps, so the 10 warps are budgeted as 12: 168 registers per thread
// is the most a launch of this shape gets (200 compiles but is refused at launch).
// Geometry of the tile a role is working on: the launch's own, or that of the tile's pixel class (MULTI).
// The slab column whose batch sums a lane of a drain warp ends up holding (see the statistics step of emit_slab).
__device__ __forceinline__ int tc_stats_col(int lane) { return (lane & 7) * 4 + (lane >> 3); }

struct TileGeo {
    int M, P, Q, kblocks, S, low_h, low_w, r0, s0, ltile;
    int64_t out_off;
    const CUtensorMap* ma;
};

// STREAM: 0 = chunked drain, 1 = streaming epilogue, 2 = streaming epilogue with eight drain warps (448 threads: two
// warps per tensor-memory lane quadrant, each taking half of the tile's columns).
constexpr int TC_STREAM8 = 2;
template <int STREAM> constexpr int tc_drain_warps() { return STREAM == TC_STREAM8 ? 8 : 4; }
template <int STREAM> constexpr int tc_threads() { return (6 + tc_drain_warps<STREAM>()) * 32; }

template <int MODE, int BN, int STAGES, bool SK, int SLABS, int BSRC, int STREAM, bool MULTI, int RESKB = 0>
__global__ void __launch_bounds__(tc_threads<STREAM>(), 1)
conv_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b0,
               const __grid_constant__ CUtensorMap tmap_b1, const __grid_constant__ CUtensorMap tmap_out,
               const __grid_constant__ CUtensorMap tmap_a3, TcParams p)
{
    static_assert(!MULTI || (MODE == TCM_FWD && !SK && STREAM == 0 && BSRC != TCB_SPLIT), "pixel classes: whole-tile forward variant on the caller's filter");
    // MULTI: the activation maps of classes 0..3 travel in the parameter slots tmap_a, tmap_b1, tmap_out, tmap_a3
    // (the split-filter map and the output map have no use there: filters are read in place, rows are scattered).
    auto tile_geo = [&](int tile) {
        TileGeo t;
        if (MULTI) {
            int c = 0;
            while (c + 1 < p.ncls && tile >= p.cls_tile0[c + 1]) c++;
            t.M = p.cls_M[c]; t.P = p.cls_P[c]; t.Q = p.cls_Q[c]; t.kblocks = p.cls_kblocks[c]; t.S = p.cls_S[c];
            t.low_h = p.cls_low_h[c]; t.low_w = p.cls_low_w[c]; t.r0 = p.cls_r0[c]; t.s0 = p.cls_s0[c];
            t.ltile = tile - p.cls_tile0[c]; t.out_off = p.cls_out[c];
            t.ma = c == 0 ? &tmap_a : c == 1 ? &tmap_b1 : c == 2 ? &tmap_out : &tmap_a3;
        } else {
            t.M = p.M; t.P = p.P; t.Q = p.Q; t.kblocks = p.kblocks; t.S = p.S; t.low_h = p.low_h; t.low_w = p.low_w;
            t.r0 = p.tap_r0; t.s0 = p.tap_s0; t.ltile = tile; t.out_off = 0; t.ma = &tmap_a;
        }
        return t;
    };
    pdl_launch_dependents();
    // Persistent: each CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ... (column tile fastest, so
    // CTAs running at the same time share activation rows in L2).  The smem pipeline and the two TMEM
    // buffers keep running across tile boundaries: the producer prefetches the next tile while the
    // drain warps still store the previous one.
    using L = TcSmem<BN, STAGES, SLABS, tc_drain_warps<STREAM>(), RESKB>;
    constexpr int DW = tc_drain_warps<STREAM>();
    constexpr int TSLOTS = L::TSLOTS;
    static_assert(RESKB == 0 || (STREAM == TC_STREAM8 && BSRC != TCB_SPLIT), "resident filters: short-K streaming variant on the caller's filter");
    // STREAM variants serve tiles of at most TC_CHUNK k-blocks with dense outputs (see dispatch_fwd)
    static_assert(STREAM == 0 || (MODE == TCM_FWD && !SK), "the streaming epilogue is a whole-tile forward variant");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full_bar = (uint64_t*)(smem + L::BAR_OFFSET);
    uint64_t* xform_bar = full_bar + STAGES;
    uint64_t* empty_bar = xform_bar + TSLOTS;
    uint64_t* tfull_bar = empty_bar + TSLOTS;
    uint64_t* tempty_bar = tfull_bar + 2;
    uint64_t* afree_bar = tempty_bar + 2;              // RESKB: the transform warps have read the stage's A tile
    uint64_t* bres_bar = afree_bar + STAGES;           // RESKB: the resident B tiles have landed
    uint32_t* tmem_slot = (uint32_t*)(bres_bar + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    TC_PROF_DECL();
    const int mt = (p.M + 127) / 128, nt = (p.N + BN - 1) / BN;
    const int total_tiles = MULTI ? p.cls_tile0[p.ncls] : mt * nt * p.splits;

    if (threadIdx.x == 32) {      // the tensor maps are kernel parameters: their fetch can start before anything else
        tma_prefetch_map(&tmap_a); tma_prefetch_map(&tmap_b0);
        if (BSRC == TCB_SPLIT && MODE == TCM_FWD) tma_prefetch_map(&tmap_b1);
        if (p.tma_store) tma_prefetch_map(&tmap_out);
        if (MULTI) { if (p.ncls > 1) tma_prefetch_map(&tmap_b1); if (p.ncls > 2) tma_prefetch_map(&tmap_out); if (p.ncls > 3) tma_prefetch_map(&tmap_a3); }
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(&full_bar[s], 1); mbar_init(&afree_bar[s], 4); }
        for (int s = 0; s < TSLOTS; s++) { mbar_init(&xform_bar[s], 4); mbar_init(&empty_bar[s], 1); }
        mbar_init(bres_bar, 1);
        for (int b = 0; b < 2; b++) { mbar_init(&tfull_bar[b], 1); mbar_init(&tempty_bar[b], DW); }
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) { tmem_alloc(tmem_slot, L::TMEM_COLS); tmem_relinquish(); }
    // barriers, tensor memory and the abort flag are on-chip state, set up while the kernel before this one in the
    // stream may still be draining; global memory is first touched below, after that kernel has completed
    pdl_wait();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        // The warp stays converged (every lane waits and computes the same coordinates); one elected lane arms
        // the barrier and issues the boxes of the k-block.
        int it = 0;
        bool ok = true;
        if (RESKB) {
            // The grid is a multiple of the column-tile count: this CTA only meets column tile blockIdx.x % nt, whose
            // filter tiles (all k-blocks) are fetched once.
            const int n0r = (int)(blockIdx.x % nt) * BN;
            if (elect_one_sync()) {
                mbar_expect_tx(bres_bar, (uint32_t)(p.kblocks * L::B_BYTES));
                for (int kb = 0; kb < p.kblocks; kb++) {
                    const int tap = kb / p.cblocks, cb = kb - tap * p.cblocks;
                    const int r = tap / p.S, sx = tap - r * p.S;
                    const int tap_real = (p.tap_r0 + p.tap_rstep * r) * p.tap_sreal + p.tap_s0 + p.tap_sstep * sx;
                    uint8_t* dst = smem + L::RES_OFFSET + kb * 2 * L::B_BYTES;
                    if (BSRC == TCB_RAW_K) {
                        tma_load_3d(dst, &tmap_b0, bres_bar, cb * 32, tap_real, n0r);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 32; j++)       // boxes past N are zero-filled by the TMA unit
                            tma_load_3d(dst + j * 4096, &tmap_b0, bres_bar, n0r + 32 * j, tap_real, cb * 32);
                    }
                }
            }
            __syncwarp();
        }
        TileWalk w;
        w.init(total_tiles, p.kblocks);
        while (ok && w.template next<SK>()) {
            const TileGeo tg = tile_geo(w.tile);
            if (MULTI) w.kb_e = tg.kblocks;
            const int tile = tg.ltile;
            const int ni = tile % nt, rest = tile / nt, mi = MULTI ? rest : rest % mt, z = MULTI ? 0 : rest / mt;
            const int m0 = mi * 128, n0 = ni * BN;
            int img = 0, base_w = 0, base_h = 0;
            if (MODE == TCM_FWD) {
                img = m0 / (tg.P * tg.Q);
                const int rem = m0 - img * (tg.P * tg.Q);
                const int p0 = rem / tg.Q, q0 = rem - p0 * tg.Q;
                base_w = q0 * p.str_w + tg.low_w; base_h = p0 * p.str_h + tg.low_h;
            }
            // WGRAD: the tile's boxes are fixed: up to four x boxes (32, 64 or 128 rows of (tap, ci) each: a box stays
            // inside one tap because its width divides C) and BN/32 dy boxes (32 output channels each)
            int box_c0[4] = {0, 0, 0, 0}, box_offw[4] = {0, 0, 0, 0}, box_offh[4] = {0, 0, 0, 0};
            uint32_t tx_bytes = 0;
            const int a_box = 1 << p.a_box_log2;
            if (MODE == TCM_WGRAD) {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int mrow = m0 + a_box * j;
                    if (a_box * j < 128 && mrow < p.M) {
                        const int tap = mrow / p.C;
                        box_c0[j] = mrow - tap * p.C;
                        const int r = tap / p.S, sx = tap - r * p.S;
                        box_offw[j] = sx * p.dil_w; box_offh[j] = r * p.dil_h;
                        tx_bytes += (uint32_t)a_box * 128u;
                    }
                }
#pragma unroll
                for (int j = 0; j < BN / 32; j++) if (n0 + 32 * j < p.N) tx_bytes += 4096u;
            }
            const int pix_begin = (MODE == TCM_WGRAD) ? z * p.kblocks * 32 : 0;
            for (int kb = w.kb_b; kb < w.kb_e; kb++, it++) {
                const int s = it % STAGES, use = it / STAGES;
                TC_PROF_T0();
                bool good = true;
                // a stage is free when the MMAs that read it have completed; with resident filters, as soon as the
                // transform warps have copied its A tile to tensor memory
                if (use > 0) good = mbar_wait(RESKB ? &afree_bar[s] : &empty_bar[s], (use - 1) & 1, abort_flag, &g_tc_status, TC_ERR_EMPTY);
                good = __all_sync(0xffffffffu, good);
                if (lane == 0) TC_PROF_ADD(0);    // producer: waiting for a free stage
                if (!good) { ok = false; break; }
                uint8_t* st = smem + s * L::STAGE_BYTES;
                if (MODE == TCM_FWD) {
                    const int tap = kb / p.cblocks, cb = kb - tap * p.cblocks;
                    const int r = tap / tg.S, sx = tap - r * tg.S;
                    if (elect_one_sync()) {
#ifdef B2C_TC_DEV
                        if (p.dbg & 64) mbar_arrive(&full_bar[s]);
                        else
#endif
                        {
                            mbar_expect_tx(&full_bar[s], (uint32_t)(RESKB ? L::A_BYTES : BSRC == TCB_SPLIT ? L::STAGE_BYTES : L::A_BYTES + L::B_BYTES));
                            tma_load_im2col_4d(st, tg.ma, &full_bar[s], cb * 32, base_w, base_h, img,
                                               (uint16_t)(sx * p.dil_w), (uint16_t)(r * p.dil_h));
                            if (RESKB) {
                                // the filter tiles are resident
                            } else if (BSRC == TCB_SPLIT) {
                                tma_load_2d(st + L::A_BYTES, &tmap_b0, &full_bar[s], kb * 32, n0);
                                tma_load_2d(st + L::A_BYTES + L::B_BYTES, &tmap_b1, &full_bar[s], kb * 32, n0);
                            } else {
                                const int tap_real = (tg.r0 + p.tap_rstep * r) * p.tap_sreal + tg.s0 + p.tap_sstep * sx;
                                if (BSRC == TCB_RAW_K) {
                                    tma_load_3d(st + L::A_BYTES, &tmap_b0, &full_bar[s], cb * 32, tap_real, n0);
                                } else {
#pragma unroll
                                    for (int j = 0; j < BN / 32; j++)       // boxes past N are zero-filled by the TMA unit
                                        tma_load_3d(st + L::A_BYTES + j * 4096, &tmap_b0, &full_bar[s], n0 + 32 * j, tap_real, cb * 32);
                                }
                            }
                        }
                    }
                } else {
                    const int pix0 = pix_begin + kb * 32;
                    const int im = pix0 / (p.P * p.Q);
                    const int rem = pix0 - im * (p.P * p.Q);
                    const int p0 = rem / p.Q, q0 = rem - p0 * p.Q;
                    const int cw = q0 * p.str_w + p.low_w, chh = p0 * p.str_h + p.low_h;
                    if (elect_one_sync()) {
#ifdef B2C_TC_DEV
                        if (p.dbg & 64) mbar_arrive(&full_bar[s]);
                        else
#endif
                        {
                        mbar_expect_tx(&full_bar[s], tx_bytes);
#pragma unroll
                        for (int j = 0; j < 4; j++)
                            if (a_box * j < 128 && m0 + a_box * j < p.M)
                                tma_load_im2col_4d(st + j * (a_box * 128), &tmap_a, &full_bar[s], box_c0[j], cw, chh, im,
                                                   (uint16_t)box_offw[j], (uint16_t)box_offh[j]);
#pragma unroll
                        for (int j = 0; j < BN / 32; j++)
                            if (n0 + 32 * j < p.N)
                                tma_load_2d(st + L::A_BYTES + j * 4096, &tmap_b0, &full_bar[s], n0 + 32 * j, pix0);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) TC_PROF_ADD(14);   // producer: TMA issue
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        // Converged warp, one elected lane issues (see elect_one_sync).
        {
            constexpr bool B_MN = MODE == TCM_WGRAD || BSRC == TCB_RAW_MN;
            constexpr uint32_t idesc = make_idesc_tf32(128, BN, 0, B_MN);
            // B tiles, K-major (FWD): rows of 128 B, 8-row groups 1024 B apart, K advances 32 B inside the row.
            // B tiles, MN-major (WGRAD): 32-row (K) boxes of 4096 B per 32 N elements, 4-row swizzle atoms of
            // 512 B, K advances by 8 rows = 1024 B.  A comes from tensor memory, K advances 8 columns.
            constexpr uint32_t LBO = B_MN ? 4096 : 0;
            constexpr uint32_t SBO = B_MN ? 512 : 1024;
            constexpr uint32_t LAYOUT = B_MN ? 1 : 2;
            constexpr uint64_t KADV = B_MN ? (1024 >> 4) : (32 >> 4);
            bool ok = true;
            int it = 0, gc = 0;
            TileWalk w;
            w.init(total_tiles, p.kblocks);
            while (ok && w.template next<SK>()) {
                if (MULTI) w.kb_e = tile_geo(w.tile).kblocks;
                for (int kb = w.kb_b; kb < w.kb_e && ok; kb++, it++) {
                    const int s = it % TSLOTS, use = it / TSLOTS;        // A slot in tensor memory (= the stage, unless the filters are resident)
                    const int b = gc & 1;
                    const bool chunk_start = ((kb - w.kb_b) % TC_CHUNK) == 0;
                    const bool chunk_end = ((kb - w.kb_b) % TC_CHUNK) == TC_CHUNK - 1 || kb == w.kb_e - 1;
                    TC_PROF_T0();
                    if (chunk_start && gc >= 2)
                        ok = mbar_wait(&tempty_bar[b], ((gc >> 1) - 1) & 1, abort_flag, &g_tc_status, TC_ERR_TEMPTY);
                    if (lane == 0) TC_PROF_ADD(1);    // MMA: waiting for a drained TMEM buffer
                    // the transform warps arrive only after they have seen the stage's TMA data land
                    if (ok) ok = mbar_wait(&xform_bar[s], use & 1, abort_flag, &g_tc_status, TC_ERR_XFORM);
                    ok = __all_sync(0xffffffffu, ok);
                    if (lane == 0) TC_PROF_ADD(3);    // MMA: waiting for the transform
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sb = RESKB ? smem_u32(smem + L::RES_OFFSET + kb * 2 * L::B_BYTES) : smem_u32(smem + s * L::STAGE_BYTES) + L::A_BYTES;
                    const uint64_t b_hi = make_smem_desc(sb, LBO, SBO, LAYOUT);
                    const uint64_t b_lo = make_smem_desc(sb + L::B_BYTES, LBO, SBO, LAYOUT);
                    const uint32_t a_hi = tmem_base + (uint32_t)(L::TMEM_A_COL + s * 64);
                    const uint32_t a_lo = a_hi + 32;
                    const uint32_t d = tmem_base + (uint32_t)(b * BN);
                    if (elect_one_sync()) {
                        // small terms first: lo*hi, hi*lo, then hi*hi
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            const uint64_t adv = (uint64_t)k * KADV;
#ifdef B2C_TC_DEV
                            if (p.dbg & 32) continue;
#endif
                            umma_tf32_ts(d, a_lo + k * 8, b_hi + adv, idesc, (!chunk_start || k > 0) ? 1u : 0u);
#ifdef B2C_TC_DEV
                            if (p.dbg & 2) continue;
#endif
                            umma_tf32_ts(d, a_hi + k * 8, b_lo + adv, idesc, 1u);
                            umma_tf32_ts(d, a_hi + k * 8, b_hi + adv, idesc, 1u);
                        }
                        umma_commit(&empty_bar[s]);
                        if (chunk_end) umma_commit(&tfull_bar[b]);
                    }
                    __syncwarp();
                    if (chunk_end) gc++;
                    if (lane == 0) TC_PROF_ADD(4);    // MMA: issue
                }
            }
        }
    } else if (warp < 6) {
        // ---------------- operand transform: a = hi + lo ----------------
        // hi = a with the low 13 mantissa bits cleared (what the tensor core reads of a float32 anyway),
        // lo = a - hi (exact).  Each thread owns one row of the A tile: it reads the row's 32 k-values from the
        // shared-memory tile and writes hi and lo into the stage's tensor-memory slot, from where the MMAs take
        // the A operand, so the A tile costs one shared-memory read in total.  In WGRAD the B tile (dy) is split
        // in shared memory as well (only lo is written: the raw tile serves as hi).
        const int quad = warp & 3;                   // TMEM lane quadrant this warp may write
        const int row = quad * 32 + lane;            // A-tile row (GEMM M index inside the tile)
        constexpr bool SPLIT_B = MODE == TCM_WGRAD || BSRC != TCB_SPLIT;    // the lo half of B is made here
        constexpr int B_VEC = SPLIT_B ? L::B_BYTES / 16 / 128 : 0;
        const int t = threadIdx.x - 64;              // 0..127
        int it = 0;
        bool ok = true;
        if (RESKB) {
            // the lo halves of the resident filter tiles, once per launch
            ok = mbar_wait(bres_bar, 0, abort_flag, &g_tc_status, TC_ERR_FULL);
            if (ok) {
                for (int kb = 0; kb < p.kblocks; kb++) {
                    const float4* b_hi = (const float4*)(smem + L::RES_OFFSET + kb * 2 * L::B_BYTES);
                    float4* b_lo = (float4*)(smem + L::RES_OFFSET + kb * 2 * L::B_BYTES + L::B_BYTES);
#pragma unroll
                    for (int i = 0; i < L::B_BYTES / 16 / 128; i++) {
                        const float4 q = b_hi[t + i * 128];
                        float4 l;
                        l.x = q.x - __uint_as_float(__float_as_uint(q.x) & 0xFFFFE000u);
                        l.y = q.y - __uint_as_float(__float_as_uint(q.y) & 0xFFFFE000u);
                        l.z = q.z - __uint_as_float(__float_as_uint(q.z) & 0xFFFFE000u);
                        l.w = q.w - __uint_as_float(__float_as_uint(q.w) & 0xFFFFE000u);
                        b_lo[t + i * 128] = l;
                    }
                }
                fence_proxy_async();
            }
        }
        TileWalk w;
        w.init(total_tiles, p.kblocks);
        while (ok && w.template next<SK>()) {
            if (MULTI) w.kb_e = tile_geo(w.tile).kblocks;
            // WGRAD: the tiles of the first row block also sum their dy tile over the pixels (the bias gradient);
            // a thread meets the same four channels of each 32-channel box in every k-block (see below)
            float4 dbacc[B_VEC / 2 + 1];
            const bool do_db = MODE == TCM_WGRAD && p.db_partial != nullptr && (w.tile / nt) % mt == 0;
#pragma unroll
            for (int i = 0; i < B_VEC / 2; i++) dbacc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int kb = w.kb_b; kb < w.kb_e; kb++, it++) {
                const int s = it % STAGES, use = it / STAGES;
                TC_PROF_T0();
                if (!mbar_wait(&full_bar[s], use & 1, abort_flag, &g_tc_status, TC_ERR_FULL)) { ok = false; break; }
                if (t == 0) TC_PROF_ADD(5);    // transform: waiting for TMA data
                const uint8_t* st = smem + s * L::STAGE_BYTES;
                // the A slot in tensor memory: the stage's own, or (resident filters) the next of a separate ring that
                // is free once the MMAs that read it have completed
                const int ts = it % TSLOTS, tuse = it / TSLOTS;
                if (RESKB && tuse > 0 && !mbar_wait(&empty_bar[ts], (tuse - 1) & 1, abort_flag, &g_tc_status, TC_ERR_EMPTY)) { ok = false; break; }
#ifdef B2C_TC_DEV
                if (p.dbg & 4) { tc_fence_before(); __syncwarp(); if (lane == 0) { if (RESKB) mbar_arrive(&afree_bar[s]); mbar_arrive(&xform_bar[ts]); } continue; }
#endif
                uint32_t v[32], h[32];
                if (MODE == TCM_FWD) {
                    // K-major 128B-swizzled tile: row r is 128 B, its 16-byte chunk c sits at chunk c ^ (r & 7)
                    const uint8_t* a_row = st + row * 128;
#pragma unroll
                    for (int c = 0; c < 8; c++) {
                        const uint4 q = *reinterpret_cast<const uint4*>(a_row + ((c ^ (row & 7)) << 4));
                        v[4 * c] = q.x; v[4 * c + 1] = q.y; v[4 * c + 2] = q.z; v[4 * c + 3] = q.w;
                    }
                } else {
                    // unswizzled boxes of [32 pixels][a_box rows]: this thread's row is a column of its box
                    const int a_box = 1 << p.a_box_log2;
                    const uint32_t* a_col = reinterpret_cast<const uint32_t*>(st + (row >> p.a_box_log2) * (a_box * 128)) + (row & (a_box - 1));
#pragma unroll
                    for (int k = 0; k < 32; k++) v[k] = a_col[k * a_box];
                }
                if (RESKB) {
                    // the A tile is in registers: the producer may refill the stage
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&afree_bar[s]);
                }
#pragma unroll
                for (int j = 0; j < 32; j++) h[j] = v[j] & 0xFFFFE000u;
                const uint32_t slot = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(L::TMEM_A_COL + ts * 64);
                tmem_st_32x32(slot, h);
#pragma unroll
                for (int j = 0; j < 32; j++) v[j] = __float_as_uint(__uint_as_float(v[j]) - __uint_as_float(h[j]));
                tmem_st_32x32(slot + 32, v);
                if (SPLIT_B && RESKB == 0) {
                    const float4* b_hi = (const float4*)(st + L::A_BYTES);
                    float4* b_lo = (float4*)(smem + s * L::STAGE_BYTES + L::A_BYTES + L::B_BYTES);
#pragma unroll
                    for (int i = 0; i < B_VEC; i++) {
                        const float4 q = b_hi[t + i * 128];
                        if (do_db) { dbacc[i >> 1].x += q.x; dbacc[i >> 1].y += q.y; dbacc[i >> 1].z += q.z; dbacc[i >> 1].w += q.w; }
                        float4 l;
                        l.x = q.x - __uint_as_float(__float_as_uint(q.x) & 0xFFFFE000u);
                        l.y = q.y - __uint_as_float(__float_as_uint(q.y) & 0xFFFFE000u);
                        l.z = q.z - __uint_as_float(__float_as_uint(q.z) & 0xFFFFE000u);
                        l.w = q.w - __uint_as_float(__float_as_uint(q.w) & 0xFFFFE000u);
                        b_lo[t + i * 128] = l;
                    }
                    fence_proxy_async();
                }
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&xform_bar[ts]);
                if (t == 0) TC_PROF_ADD(6);    // transform: work
            }
            if (MODE == TCM_WGRAD && do_db && ok) {
                // Float4 number t + 128 i of the B region is box i/2, pixel row t/8 + 16 (i & 1), 16-byte chunk t & 7.
                // The box layout XORs the 32-byte atom index (chunk >> 1) with (row & 3), so the lane's channels are
                // chunk ((c >> 1) ^ rr) * 2 + (c & 1) with c = lane & 7, rr = (lane >> 3) & 3: the four lanes that hold
                // one chunk differ by lane ^ (m << 3 | m << 1), m = 1..3.  After the two exchange steps lanes 0-7
                // (rr = 0: chunk = c) hold the warp's sums over its 8 pixel rows of every k-block.
                const int ni = w.tile % nt, z = (w.tile / nt) / mt;
#pragma unroll
                for (int bx = 0; bx < B_VEC / 2; bx++) {
                    float4 v = dbacc[bx];
#pragma unroll
                    for (int m = 1; m <= 2; m <<= 1) {
                        const int mask = (m << 3) | (m << 1);
                        v.x += __shfl_xor_sync(0xffffffffu, v.x, mask); v.y += __shfl_xor_sync(0xffffffffu, v.y, mask);
                        v.z += __shfl_xor_sync(0xffffffffu, v.z, mask); v.w += __shfl_xor_sync(0xffffffffu, v.w, mask);
                    }
                    const int n = ni * BN + bx * 32;
                    if (lane < 8 && n < p.N)
                        *reinterpret_cast<float4*>(p.db_partial + ((size_t)z * 4 + (warp - 2)) * p.N + n + lane * 4) = v;
                }
            }
        }
    } else {
        // ---------------- drain of the partial sums, then epilogue ----------------
        // Each chunk of TC_CHUNK k-blocks is accumulated in tensor memory from zero and added here in
        // float32 round-to-nearest; the tensor core's own accumulate step truncates, and its bias
        // grows with the number of accumulations, so it is kept to one chunk.
        const int quad = warp & 3;                       // TMEM lane quadrant this warp may read
        bool ok = true;
        int gc = 0, ecount = 0;
        // column slabs of a tile this warp sends out: all BN / 32, or its half of them with eight drain warps
        constexpr int NSLAB = BN / 32 / (DW / 4);
        const int cbeg = ((warp - 6) >> 2) * NSLAB;
        float cs0[NSLAB], cs1[NSLAB];                    // batch statistics summed over this CTA's tiles (stats_cta)
#pragma unroll
        for (int i = 0; i < NSLAB; i++) cs0[i] = cs1[i] = 0.f;
        TileWalk w;
        w.init(total_tiles, p.kblocks);
        while (ok && w.template next<SK>()) {
            const TileGeo tg = tile_geo(w.tile);
            if (MULTI) w.kb_e = tg.kblocks;
            const int tile = tg.ltile;
            const int ni = tile % nt, rest = tile / nt, mi = MULTI ? rest : rest % mt, z = MULTI ? 0 : rest / mt;
            const int m0 = mi * 128, n0 = ni * BN;
            // One 32-row x 32-column slab of the tile on its way out (dense outputs): epilogue steps, staging in a
            // 128B-swizzled slab (conflict-free float4 writes), TMA store (whole rows, asynchronous, rows >= M and
            // columns >= N clipped; SLABS slabs per warp rotate so the warp never waits on HBM), and the slab's batch
            // statistics when asked for.
            uint8_t* ebuf = smem + L::EPI_OFFSET + (warp - 6) * (SLABS * 4096);
            float st0[NSLAB], st1[NSLAB];                               // batch statistics of the tile's slabs
            TC_PROF_T0();
            auto emit_slab = [&](float* a, int cc, int i) {      // slab cc of the tile, number i of this warp's slabs
                uint8_t* buf = ebuf + (ecount % SLABS) * 4096;
                if (MODE == TCM_FWD && p.epi) tc_epilogue_math(p, n0 + cc * 32, a);
                if (threadIdx.x == 192) TC_PROF_ADD(8);     // drain: tensor-memory loads, adds, epilogue arithmetic
                if (lane == 0) tma_store_wait_read<SLABS - 1>();     // the store that last read this slab is done
                __syncwarp();
                if (threadIdx.x == 192) TC_PROF_ADD(10);    // drain: waiting for a free staging slab
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    *reinterpret_cast<float4*>(buf + lane * 128 + ((((j >> 2) ^ (lane & 7))) << 4)) = make_float4(a[j], a[j + 1], a[j + 2], a[j + 3]);
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                    if (MODE == TCM_FWD) tma_store_2d(&tmap_out, buf, n0 + cc * 32, m0 + quad * 32);
                    else tma_store_3d(&tmap_out, buf, n0 + cc * 32, m0 + quad * 32, z);
                    tma_store_commit();
                }
                if (threadIdx.x == 192) TC_PROF_ADD(9);     // drain: staging writes, fence, store issue
                if (MODE == TCM_FWD && p.stats) {
                    // Column sums of the slab over the rows that exist, read back from the staging slab: lane
                    // (rg = lane / 8, c4 = lane % 8) takes columns 4 c4 .. 4 c4 + 3 of rows rg, rg + 4, .. (one float4 each:
                    // the eight lanes of a row group read one whole 128-byte row, no bank conflicts), the four row groups
                    // are added by two exchange steps that also hand every lane one column: lane keeps column
                    // 4 c4 + rg (tc_stats_col).  The sums wait in registers until the tile's last slab is on its way.
                    const int valid = p.M - (m0 + quad * 32);
                    const int rg = lane >> 3, c4 = lane & 7;
                    float4 q[8];
#pragma unroll
                    for (int r = 0; r < 8; r++) {
                        const int row = rg + 4 * r;
                        const uint32_t addr = smem_u32(buf) + row * 128 + ((c4 ^ (row & 7)) << 4);
                        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(q[r].x), "=f"(q[r].y), "=f"(q[r].z), "=f"(q[r].w) : "r"(addr));
                    }
                    float4 t0 = make_float4(0.f, 0.f, 0.f, 0.f), t1 = t0;
#pragma unroll
                    for (int r = 0; r < 8; r++) {
                        float4 u = q[r];
                        if (rg + 4 * r >= valid) u = make_float4(0.f, 0.f, 0.f, 0.f);       // rows past M count as zeros
                        t0.x += u.x; t0.y += u.y; t0.z += u.z; t0.w += u.w;
                        t1.x = fmaf(u.x, u.x, t1.x); t1.y = fmaf(u.y, u.y, t1.y); t1.z = fmaf(u.z, u.z, t1.z); t1.w = fmaf(u.w, u.w, t1.w);
                    }
                    const bool up = (lane & 16) != 0, odd = (lane & 8) != 0;
                    // step 1 (partner lane ^ 16): the lower lane keeps columns 0, 1 of the four, the upper one 2, 3
                    float k0 = up ? t0.z : t0.x, k1 = up ? t0.w : t0.y, g0 = up ? t0.x : t0.z, g1 = up ? t0.y : t0.w;
                    float m0s = up ? t1.z : t1.x, m1s = up ? t1.w : t1.y, h0 = up ? t1.x : t1.z, h1 = up ? t1.y : t1.w;
                    k0 += __shfl_xor_sync(0xffffffffu, g0, 16); k1 += __shfl_xor_sync(0xffffffffu, g1, 16);
                    m0s += __shfl_xor_sync(0xffffffffu, h0, 16); m1s += __shfl_xor_sync(0xffffffffu, h1, 16);
                    // step 2 (partner lane ^ 8): one column each
                    float s0 = odd ? k1 : k0, e0 = odd ? k0 : k1, s1 = odd ? m1s : m0s, e1 = odd ? m0s : m1s;
                    s0 += __shfl_xor_sync(0xffffffffu, e0, 8); s1 += __shfl_xor_sync(0xffffffffu, e1, 8);
                    st0[i] = s0; st1[i] = s1;
                    if (threadIdx.x == 192) TC_PROF_ADD(11);    // drain: batch statistics
                }
                ecount++;
            };
            auto store_stats = [&]() {
                if (MODE == TCM_FWD && p.stats && p.stats_cta && m0 + quad * 32 < p.M) {
                    // the grid is a multiple of the column-tile count, so every tile of this CTA has the same n0
#pragma unroll
                    for (int i = 0; i < NSLAB; i++)
                        if (n0 + (cbeg + i) * 32 < p.N) { cs0[i] += st0[i]; cs1[i] += st1[i]; }
                } else if (MODE == TCM_FWD && p.stats && m0 + quad * 32 < p.M) {
                    // row (m / 32) of the statistics: the block's two rows of sums, 128 contiguous bytes per slab
                    const int col = tc_stats_col(lane);
                    float* srow = p.stats + ((size_t)((m0 >> 5) + quad) * 2) * p.N + n0 + cbeg * 32 + col;
#pragma unroll
                    for (int i = 0; i < NSLAB; i++)
                        if (n0 + (cbeg + i) * 32 + col < p.N) { __stcg(srow + i * 32, st0[i]); __stcg(srow + i * 32 + p.N, st1[i]); }
                }
            };
            if constexpr (STREAM != 0) {
                // Short K loops: the tile is one chunk in tensor memory and the epilogue, not the tensor pipe, sets the
                // pace.  The drain warp takes 32 columns at a time straight from tensor memory (the next 32 already in
                // flight) and sends them out, so it never holds a whole row of the tile in registers.
                const int b = gc & 1;
                TC_PROF_RESET();
                ok = mbar_wait(&tfull_bar[b], (gc >> 1) & 1, abort_flag, &g_tc_status, TC_ERR_TFULL);
                if (threadIdx.x == 192) TC_PROF_ADD(7);
                if (!ok) break;
                tc_fence_after();
                const uint32_t tsrc = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(b * BN);
                float a[2][32];
                tmem_ld_32x32_f(tsrc + (uint32_t)(cbeg * 32), a[0]);
#pragma unroll
                for (int i = 0; i < NSLAB; i++) {
                    const int cc = cbeg + i;
                    tmem_ld_wait();
                    if (i + 1 < NSLAB) tmem_ld_32x32_f(tsrc + (uint32_t)((cc + 1) * 32), a[(i + 1) & 1]);
                    else {
                        // every column this warp takes is in registers: the tensor core may have the buffer back
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&tempty_bar[b]);
                    }
                    if (n0 + cc * 32 < p.N && m0 + quad * 32 < p.M) emit_slab(a[i & 1], cc, i);
                }
                gc++;
                store_stats();
            } else {
            const int nchunks = (w.kb_e - w.kb_b + TC_CHUNK - 1) / TC_CHUNK;
            float acc[BN];
            for (int c = 0; c < nchunks && ok; c++, gc++) {
                const int b = gc & 1;
                TC_PROF_RESET();
                ok = mbar_wait(&tfull_bar[b], (gc >> 1) & 1, abort_flag, &g_tc_status, TC_ERR_TFULL);
                if (threadIdx.x == 192) TC_PROF_ADD(7);    // drain: waiting for a finished chunk
                if (!ok) break;
                tc_fence_after();
                const uint32_t tsrc = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(b * BN);
                if (c == 0) {
                    // first chunk: straight into the accumulators, all loads in flight before the one wait
#pragma unroll
                    for (int cc = 0; cc < BN / 32; cc++) tmem_ld_32x32_f(tsrc + (uint32_t)(cc * 32), &acc[cc * 32]);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int cc = 0; cc < BN / 32; cc++) {
                        uint32_t r[32];
                        tmem_ld_32x32(tsrc + (uint32_t)(cc * 32), r);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; j++) acc[cc * 32 + j] += __uint_as_float(r[j]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&tempty_bar[b]);
                if (threadIdx.x == 192) TC_PROF_ADD(8);    // drain: TMEM load + add
            }
            if (SK && ok) {
                const int row = quad * 32 + lane;
                if (w.kb_b > 0) {
                    // a later part of a tile another CTA started: hand the partial tile over, no epilogue
                    float4* slot = reinterpret_cast<float4*>(p.sk_partial + (size_t)blockIdx.x * (128 * BN)) + row;
#pragma unroll
                    for (int j = 0; j < BN; j += 4) slot[(j >> 2) * 128] = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
                    __threadfence();
                    __syncwarp();
                    if (lane == 0) st_release_gpu(&p.sk_flags[blockIdx.x * 4 + quad], 1);
                    continue;
                }
                if (w.kb_e < p.kblocks) {
                    // this CTA started the tile and its range ended inside it: the following CTAs hold the rest
                    const long long total = (long long)total_tiles * p.kblocks;
                    const long long tile_end = (long long)(tile + 1) * p.kblocks;
                    for (int c2 = blockIdx.x + 1; c2 < (int)gridDim.x && ok; c2++) {
                        if (TileWalk::range_begin(total, c2, gridDim.x) >= tile_end) break;
                        int got = 1;
                        if (lane == 0) {
                            const int* flag = &p.sk_flags[c2 * 4 + quad];
                            long long t0 = 0;
                            uint32_t tries = 0;
                            while (ld_acquire_gpu(flag) == 0) {
                                if ((++tries & 15u) == 0) {
                                    const long long now = clock64();
                                    if (*abort_flag) { got = 0; break; }
                                    if (t0 == 0) t0 = now;
                                    else if (now - t0 > TC_WAIT_CYCLES) { *abort_flag = 1; atomicCAS(&g_tc_status, 0, TC_ERR_PARTIAL); got = 0; break; }
                                }
                            }
                        }
                        got = __shfl_sync(0xffffffffu, got, 0);
                        if (!got) { ok = false; break; }
                        __threadfence();
                        // this warp is the flag's only reader: once seen, it goes back to zero for the next launch
                        if (p.sk_selfclean && lane == 0) p.sk_flags[c2 * 4 + quad] = 0;
                        const float4* slot = reinterpret_cast<const float4*>(p.sk_partial + (size_t)c2 * (128 * BN)) + row;
#pragma unroll
                        for (int j = 0; j < BN; j += 4) {
                            const float4 q = __ldcg(slot + (j >> 2) * 128);
                            acc[j] += q.x; acc[j + 1] += q.y; acc[j + 2] += q.z; acc[j + 3] += q.w;
                        }
                    }
                }
            }
            TC_PROF_RESET();
            // Epilogue. A thread owns one output row, but a warp writing 32 different rows per store would
            // touch 32 cache lines with 16 bytes each; the values go through a per-warp smem tile instead so
            // that every store instruction writes whole 128-byte row segments (8 lanes per row, 4 rows).
            const int m = m0 + quad * 32 + lane;
            int64_t my_off = -1;
            int zmask = 0;                       // zfill: which of the row's three neighbour pixels exist
            if (m < tg.M) {
                if (MODE == TCM_FWD) {
                    const int img = m / (tg.P * tg.Q);
                    const int rem = m - img * (tg.P * tg.Q);
                    const int pi = rem / tg.Q, qi = rem - pi * tg.Q;
                    my_off = tg.out_off + img * p.o_sn + pi * p.o_sh + qi * p.o_sw;
                    if (p.zfill) zmask = (2 * qi + 1 < p.z_W ? 1 : 0) | (2 * pi + 1 < p.z_H ? 2 : 0);
                } else {
                    my_off = ((int64_t)z * p.M + m) * p.N;
                }
            }
            if (ok && p.tma_store) {
#pragma unroll
                for (int cc = 0; cc < BN / 32; cc++)
                    if (n0 + cc * 32 < p.N && m0 + quad * 32 < p.M) emit_slab(&acc[cc * 32], cc, cc);     // slabs wholly outside the output are skipped
                store_stats();
            } else if (ok) {
                float* stage = (float*)(smem + L::EPI_OFFSET) + (warp - 6) * (SLABS * 4096 / 4);
#pragma unroll
                for (int cc = 0; cc < BN / 32; cc++) {
                    if (n0 + cc * 32 < p.N) {
                        if (MODE == TCM_FWD && p.epi) tc_epilogue_math(p, n0 + cc * 32, &acc[cc * 32]);
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            *reinterpret_cast<float4*>(stage + lane * 36 + j) =
                                make_float4(acc[cc * 32 + j], acc[cc * 32 + j + 1], acc[cc * 32 + j + 2], acc[cc * 32 + j + 3]);
                        __syncwarp();
#pragma unroll
                        for (int i = 0; i < 8; i++) {
                            const int r = i * 4 + (lane >> 3), c4 = (lane & 7) * 4;
                            const int64_t off_r = __shfl_sync(0xffffffffu, my_off, r);
                            const int zm = __shfl_sync(0xffffffffu, zmask, r);
                            const int n = n0 + cc * 32 + c4;
                            if (off_r >= 0 && n < p.N) {
                                *reinterpret_cast<float4*>(p.out + off_r + n) = *reinterpret_cast<const float4*>(stage + r * 36 + c4);
                                if (MODE == TCM_FWD && zm) {
                                    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
                                    if (zm & 1) *reinterpret_cast<float4*>(p.out + off_r + p.z_w + n) = zero;
                                    if (zm & 2) *reinterpret_cast<float4*>(p.out + off_r + p.z_h + n) = zero;
                                    if (zm == 3) *reinterpret_cast<float4*>(p.out + off_r + p.z_h + p.z_w + n) = zero;
                                }
                            }
                        }
                        __syncwarp();
                    }
                }
            }
            if (threadIdx.x == 192) TC_PROF_ADD(9);        // drain: epilogue
            }   // chunked drain
        }
        if (MODE == TCM_FWD && !SK && !MULTI && p.stats && p.stats_cta && ok) {
            // One row of sums per (group of nt CTAs, row quadrant): the nt CTAs of a group hold the nt column tiles.
            const int n0 = (int)(blockIdx.x % nt) * BN;
            const int col = tc_stats_col(lane);
            float* srow = p.stats + ((size_t)((blockIdx.x / nt) * 4 + quad) * 2) * p.N + n0 + cbeg * 32 + col;
#pragma unroll
            for (int i = 0; i < NSLAB; i++)
                if (n0 + (cbeg + i) * 32 + col < p.N) { __stcg(srow + i * 32, cs0[i]); __stcg(srow + i * 32 + p.N, cs1[i]); }
        }
        if (p.tma_store && lane == 0) tma_store_wait_read<0>();   // the slabs stay allocated until the last store has read them
    }
    TC_PROF_FLUSH();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, L::TMEM_COLS); }
}

// Second stage of the weight gradient: fixed-order sum of the per-split partial tiles, written in the
// caller's filter layout.
struct WgradReduceParams { int M, N, C, S, splits; int64_t sk, sc, sr, ss; int Mreal; };

template <int ROWS>
__global__ void __launch_bounds__(256) tc_wgrad_reduce_kernel(WgradReduceParams p, const float* __restrict__ partial, float* __restrict__ dw,
                                                              const float* __restrict__ db_partial, float* __restrict__ db)
{
    pdl_prologue();
    // bias gradient: the [splits][4] per-channel sums, added in a fixed order (first block row only)
    if (db && blockIdx.y == 0) {
        const int n = blockIdx.x * 32 + threadIdx.x;
        if (threadIdx.y == 0 && n < p.N) {
            float v = 0.f;
            for (int i = 0; i < p.splits * 4; i++) v += __ldcg(db_partial + (size_t)i * p.N + n);
            db[n] = v;
        }
    }
    // A block owns 8 * ROWS rows (tap, ci) x 32 output channels.  Thread (x, y) adds, in split order, the partials of
    // column n0 + x for rows y, y + 8, ... (loads of a warp cover 128 contiguous bytes; ROWS rows x 16 / ROWS splits
    // at a time are independent loads).  ROWS = 4 for large filters; ROWS = 1 makes four times the blocks when the
    // filter is small and the splits are many (the sum over the splits is the long loop then).  The sums leave along
    // whichever axis is contiguous in the caller's filter layout: output channels as they are, (tap, ci) rows through
    // a transposing shared-memory tile.
    constexpr int TR = 8 * ROWS, U = 16 / ROWS;
    __shared__ float tile[TR][33];
    const int m0 = blockIdx.y * TR, n0 = blockIdx.x * 32;
    const int64_t plane = (int64_t)p.M * p.N;
    const int n = n0 + threadIdx.x;
    float v[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; r++) v[r] = 0.f;
    if (n < p.N) {
        const float* src = partial + (int64_t)(m0 + threadIdx.y) * p.N + n;
        bool in[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; r++) in[r] = m0 + threadIdx.y + 8 * r < p.M;
        int z = 0;
        for (; z + U <= p.splits; z += U) {
            float q[U][ROWS];
#pragma unroll
            for (int u = 0; u < U; u++)
#pragma unroll
                for (int r = 0; r < ROWS; r++) q[u][r] = in[r] ? __ldcg(src + (int64_t)(z + u) * plane + (int64_t)(8 * r) * p.N) : 0.f;
#pragma unroll
            for (int u = 0; u < U; u++)
#pragma unroll
                for (int r = 0; r < ROWS; r++) v[r] += q[u][r];
        }
        for (; z < p.splits; z++)
#pragma unroll
            for (int r = 0; r < ROWS; r++) v[r] += in[r] ? __ldcg(src + (int64_t)z * plane + (int64_t)(8 * r) * p.N) : 0.f;
    }
    if (p.sk == 1) {
        // output channels contiguous: store the row segments as they are
#pragma unroll
        for (int r = 0; r < ROWS; r++) {
            const int m = m0 + threadIdx.y + 8 * r;
            if (m < p.Mreal && n < p.N) {            // rows >= Mreal: zero padding of a lowered few-channel layer
                const int tap = m / p.C, c = m - tap * p.C, rr = tap / p.S, s = tap - rr * p.S;
                dw[c * p.sc + rr * p.sr + s * p.ss + n] = v[r];
            }
        }
        return;
    }
#pragma unroll
    for (int r = 0; r < ROWS; r++) tile[threadIdx.y + 8 * r][threadIdx.x] = v[r];
    __syncthreads();
    // lanes now run along the rows: thread (x, y) with x < TR writes row m0 + x for columns y, y + 8, y + 16, y + 24
    const int m = m0 + threadIdx.x;
    if (threadIdx.x >= TR || m >= p.Mreal) return;
    const int tap = m / p.C, c = m - tap * p.C, rr = tap / p.S, s = tap - rr * p.S;
    float* d = dw + c * p.sc + rr * p.sr + s * p.ss;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int nn = n0 + threadIdx.y + 8 * j;
        if (nn < p.N) d[(int64_t)nn * p.sk] = tile[threadIdx.x][threadIdx.y + 8 * j];
    }
}

// The same sum for small filters cut into very many splits (a 64 x 64 filter summed over 148 pixel ranges): a block
// owns one row x 32 output channels and its 8 thread rows share the splits (thread row y adds splits y, y + 8, ... in
// order, then the 8 partial sums are added in thread-row order: a fixed order again).
__global__ void __launch_bounds__(256) tc_wgrad_reduce_deep_kernel(WgradReduceParams p, const float* __restrict__ partial, float* __restrict__ dw,
                                                                   const float* __restrict__ db_partial, float* __restrict__ db)
{
    pdl_prologue();
    __shared__ float part[8][33];
    const int n = blockIdx.x * 32 + threadIdx.x, m = blockIdx.y;
    if (db && blockIdx.y == 0) {
        // bias gradient: [splits * 4] row sums per channel, shared among the thread rows the same way
        float v = 0.f;
        if (n < p.N) for (int i = threadIdx.y; i < p.splits * 4; i += 8) v += __ldcg(db_partial + (size_t)i * p.N + n);
        part[threadIdx.y][threadIdx.x] = v;
        __syncthreads();
        if (threadIdx.y == 0 && n < p.N) {
            float t = 0.f;
#pragma unroll
            for (int y = 0; y < 8; y++) t += part[y][threadIdx.x];
            db[n] = t;
        }
        __syncthreads();
    }
    const int64_t plane = (int64_t)p.M * p.N;
    float v = 0.f;
    if (n < p.N) {
        const float* src = partial + (int64_t)m * p.N + n;
        int z = threadIdx.y;
        for (; z + 56 < p.splits; z += 64) {
            float q[8];
#pragma unroll
            for (int u = 0; u < 8; u++) q[u] = __ldcg(src + (int64_t)(z + 8 * u) * plane);
#pragma unroll
            for (int u = 0; u < 8; u++) v += q[u];
        }
        for (; z < p.splits; z += 8) v += __ldcg(src + (int64_t)z * plane);
    }
    part[threadIdx.y][threadIdx.x] = v;
    __syncthreads();
    if (threadIdx.y != 0 || n >= p.N || m >= p.Mreal) return;
    float t = 0.f;
#pragma unroll
    for (int y = 0; y < 8; y++) t += part[y][threadIdx.x];
    const int tap = m / p.C, c = m - tap * p.C, rr = tap / p.S, s = tap - rr * p.S;
    dw[(int64_t)n * p.sk + c * p.sc + rr * p.sr + s * p.ss] = t;
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
static bool make_map_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                        CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_128B)
{
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * sizeof(float)};
    cuuint32_t box[2] = {32, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return g_encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// NHWC activation tensor (n, h, w, c) seen through an im2col window of `pixels` consecutive window
// positions x 32 channels per load. The window's first position sits at (low_h, low_w); it has
// `cnt_h` x `cnt_w` positions per image before the traversal stride is applied. Corners in (w, h) order.
static bool make_map_im2col(CUtensorMap* map, const void* base, int n, int h, int w, int c, int low_h, int low_w,
                            int cnt_h, int cnt_w, int str_h, int str_w, uint32_t pixels,
                            CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_128B, uint32_t channels = 32)
{
    cuuint64_t dims[4] = {(cuuint64_t)c, (cuuint64_t)w, (cuuint64_t)h, (cuuint64_t)n};
    cuuint64_t strides[3] = {(cuuint64_t)c * 4, (cuuint64_t)w * c * 4, (cuuint64_t)h * w * c * 4};
    int lower[2] = {low_w, low_h};
    int upper[2] = {cnt_w - w + low_w, cnt_h - h + low_h};
    for (int i = 0; i < 2; i++) if (lower[i] < -128 || lower[i] > 127 || upper[i] < -128 || upper[i] > 127) return false;
    cuuint32_t estr[4] = {1, (cuuint32_t)str_w, (cuuint32_t)str_h, 1};
    return g_encode_im2col(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(base), dims, strides, lower, upper,
                           channels, pixels, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// One parity class of a strided data gradient along one axis: output positions o = str*i + a.
// The filter taps that reach them are r = a + pad - str*delta (dilation 1); delta runs over
// [dmin, dmin + cnt).  cnt == 0: no tap reaches the class (its outputs are zero).
struct AxisClass { int cnt, dmin, r0, out_cnt; };
static AxisClass axis_class(int a, int str, int pad, int k, int in_len)
{
    AxisClass c{0, 0, 0, 0};
    c.out_cnt = in_len > a ? (in_len - a + str - 1) / str : 0;
    int dmin = 1 << 30, dmax = -(1 << 30);
    for (int r = 0; r < k; r++) {
        int t = a + pad - r;
        if (t % str != 0) continue;                    // C remainder: exact for negative t too
        int d = t / str;
        if (d < dmin) dmin = d;
        if (d > dmax) dmax = d;
    }
    if (dmax < dmin) return c;
    c.cnt = dmax - dmin + 1; c.dmin = dmin; c.r0 = a + pad - str * dmin;
    return c;
}

// Few-channel layers run through the written-out im2row matrix (see tc_lower_kernel).
static int lowered_kp(const Geo& g) { return (int)((g.K + 31) / 32 * 32); }
static bool lowered_ok(const Geo& g)
{
    if (g.ci % 32 == 0 || g.ci > 16) return false;
    if (g.K > 1024) return false;
    return (int64_t)g.M * lowered_kp(g) * 4 <= (int64_t)3 << 30;
}

static bool tc_supported_nhwc(const Geo& g, int pass)
{
    if (g.dtype != B2C_F32 || g.layout != B2C_LAYOUT_NHWC || g.engine == B2C_ENGINE_FMA) return false;
    if (g.vstr > 8 || g.hstr > 8) return false;
    if ((g.kh - 1) * g.vdil > 255 || (g.kw - 1) * g.hdil > 255 || g.vpad > 127 || g.hpad > 127) return false;
    if (pass == B2C_PASS_FPROP) return (g.ci % 32 == 0 || lowered_ok(g)) && g.co % 4 == 0;
    if (pass == B2C_PASS_DGRAD) {
        if (g.co % 32 || g.ci % 4) return false;
        if (g.vstr == 1 && g.hstr == 1) return (g.kh - 1) * g.vdil - g.vpad >= -127 && (g.kw - 1) * g.hdil - g.hpad >= -127;
        return g.vdil == 1 && g.hdil == 1;             // strided: parity-class decomposition, dilation 1 only
    }
    return (g.ci % 32 == 0 || lowered_ok(g)) && g.co % 32 == 0;
}

// Function attributes and the SM count belong to a device, not to the process: both are kept per device ordinal
// (the device current at the call), so a process that drives several GPUs sets each one up.
#define B2C_MAX_DEVICES 64
static int current_device()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= B2C_MAX_DEVICES) dev = 0;
    return dev;
}
struct PerDeviceOnce {
    std::mutex m;
    bool done[B2C_MAX_DEVICES] = {};
    // Runs fn() the first time it is called with a given device current; returns fn's error (and retries next time).
    template <typename Fn> cudaError_t run(Fn fn) {
        const int dev = current_device();
        std::lock_guard<std::mutex> lock(m);
        if (done[dev]) return cudaSuccess;
        cudaError_t e = fn();
        if (e == cudaSuccess) done[dev] = true;
        return e;
    }
};

static int tc_sm_count()
{
    static int sm_count[B2C_MAX_DEVICES] = {};
    static std::mutex m;
    const int dev = current_device();
    std::lock_guard<std::mutex> lock(m);
    if (!sm_count[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        sm_count[dev] = n;
    }
    return sm_count[dev];
}
// The bank of synchronisation words of `st` on the current device, or null when all banks belong to other streams.
// In host code g_tc_sync is only a handle for the runtime: the device address is looked up once per device.
static unsigned int* tc_sync_bank(cudaStream_t st)
{
    static std::mutex m;
    static unsigned int* base[B2C_MAX_DEVICES] = {};
    static cudaStream_t owner[B2C_MAX_DEVICES][TC_SYNC_BANKS];
    static int owners[B2C_MAX_DEVICES] = {};
    const int dev = current_device();
    std::lock_guard<std::mutex> lock(m);
    if (!base[dev]) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_tc_sync) != cudaSuccess || !ptr) { cudaGetLastError(); return nullptr; }
        base[dev] = (unsigned int*)ptr;
    }
    for (int i = 0; i < owners[dev]; i++)
        if (owner[dev][i] == st) return base[dev] + (size_t)i * TC_SYNC_WORDS;
    if (owners[dev] == TC_SYNC_BANKS) return nullptr;
    owner[dev][owners[dev]] = st;
    return base[dev] + (size_t)(owners[dev]++) * TC_SYNC_WORDS;
}

// Whole tiles against balanced ranges: balanced mode is taken when its cost estimate is below this share of the plain
// one (B2C_TC_BALANCE overrides it, for experiments).
static double tc_balance_threshold()
{
    static double v = -1.0;
    if (v < 0.0) { const char* e = getenv("B2C_TC_BALANCE"); v = e ? atof(e) : 0.85; }
    return v;
}

// Balanced mode scratch: 4 flags per CTA (padded to 4 KB) and one 128 x 128 float partial tile per CTA.
static size_t sk_flag_bytes() { return align_up((size_t)tc_sm_count() * 4 * sizeof(int), 4096); }
static size_t sk_bytes() { return sk_flag_bytes() + (size_t)tc_sm_count() * 128 * 128 * sizeof(float); }

static size_t filter_split_bytes(const Geo& g, int pass)
{
    int rows = pass == B2C_PASS_FPROP ? g.co : g.ci;
    int C = pass == B2C_PASS_FPROP ? g.ci : g.co;
    return align_up((size_t)rows * g.kh * g.kw * C * sizeof(float), 1024);
}

struct WgradPlan { int splits, kblocks, bn; };
// The pixel axis is cut into `splits` ranges of `kblocks` 32-pixel blocks; tiles x splits work items run on one
// persistent CTA per SM.  The split count minimises a cost in k-block units: rounds of the CTA grid x (k-blocks per
// item + a fixed per-item cost for pipeline fill, drain and the partial-tile store) + the second-stage reduce, whose
// traffic grows with the split count.
static WgradPlan wgrad_plan(const Geo& g)
{
    WgradPlan pl;
    pl.bn = g.co <= 64 ? 64 : 128;
    const int64_t Krows = g.ci % 32 == 0 ? g.K : lowered_kp(g);
    const int64_t tiles = ((Krows + 127) / 128) * ((g.co + pl.bn - 1) / pl.bn);
    const int64_t blocks = (g.M + 31) / 32;
    const double reduce_per_split = (double)Krows * g.co * 4.0 / 5e12 / 0.6e-6;   // k-block units (0.6 us each)
    double best = 0.0;
    const int64_t G = tc_sm_count();
    pl.splits = 1; pl.kblocks = (int)blocks;
    for (int64_t s = 1; s <= 512 && s <= blocks; s++) {
        const int64_t kb = (blocks + s - 1) / s;
        if ((blocks + kb - 1) / kb != s) continue;       // same k-blocks per split as a smaller count
        if (kb < 4 && s > 1) break;
        const int64_t rounds = (tiles * s + G - 1) / G;
        const double cost = (double)rounds * (double)(kb + 6) + (double)s * reduce_per_split;
        if (s == 1 || cost < best) { best = cost; pl.splits = (int)s; pl.kblocks = (int)kb; }
    }
    return pl;
}

// A 1x1 stride-1 weight gradient whose (tap, ci) rows fill at most half of a 128-row MMA (ci <= 64) while co would fill
// it: the roles of x and dy are exchanged (dw^T = dy^T x, computed as the weight gradient of the layer with ci and co
// exchanged, x in the place of dy), and the second stage writes dw through exchanged filter strides.  The bias
// gradient comes out of the B-operand path, which then holds x: layers that ask for it keep the plain form.
static bool wgrad_swap_ok(const Geo& g)
{
    return g.kh == 1 && g.kw == 1 && g.vstr == 1 && g.hstr == 1 && g.vpad == 0 && g.hpad == 0 &&
           g.ci % 32 == 0 && g.ci <= 64 && g.co % 32 == 0 && g.co >= 128;
}
static Geo wgrad_swapped(const Geo& g)
{
    Geo q = g;
    q.ci = g.co; q.co = g.ci; q.K = q.ci;
    return q;
}

static size_t tc_workspace_bytes_nhwc(const Geo& g, int pass)
{
    if (pass == B2C_PASS_WGRAD && wgrad_swap_ok(g)) {
        // either form may run (the bias gradient decides at the call): room for both
        const size_t a = tc_workspace_bytes_nhwc(wgrad_swapped(g), pass);      // not exchanged again: its co is at most 64
        const WgradPlan pl = wgrad_plan(g);
        const size_t b = align_up((size_t)pl.splits * g.K * g.co * sizeof(float), 1024) + 2048 + align_up((size_t)pl.splits * 4 * g.co * sizeof(float), 1024);
        return a > b ? a : b;
    }
    const bool low = g.ci % 32 != 0;
    const size_t lowered = low ? align_up((size_t)g.M * lowered_kp(g) * sizeof(float), 1024) : 0;
    if (pass == B2C_PASS_FPROP && low) return lowered + 2 * align_up((size_t)g.co * lowered_kp(g) * sizeof(float), 1024) + 2048;
    if (pass == B2C_PASS_FPROP || pass == B2C_PASS_DGRAD) return 2 * filter_split_bytes(g, pass) + 1024 + sk_bytes();
    WgradPlan pl = wgrad_plan(g);
    const size_t Krows = low ? (size_t)lowered_kp(g) : (size_t)g.K;
    return lowered + align_up((size_t)pl.splits * Krows * g.co * sizeof(float), 1024) + 2048 +
           align_up((size_t)pl.splits * 4 * g.co * sizeof(float), 1024);
}

template <int MODE, int BN, int STAGES, bool SK, int SLABS, int BSRC, int STREAM = 0, bool MULTI = false, int RESKB = 0>
static int launch_tc(const CUtensorMap& ma, const CUtensorMap& mb0, const CUtensorMap& mb1, const CUtensorMap& mo, const TcParams& p, int splits, cudaStream_t st,
                     const CUtensorMap* ma3 = nullptr)
{
    using L = TcSmem<BN, STAGES, SLABS, tc_drain_warps<STREAM>(), RESKB>;
    static PerDeviceOnce attr;
    {
        cudaError_t e = attr.run([] { return cudaFuncSetAttribute(conv_tc_kernel<MODE, BN, STAGES, SK, SLABS, BSRC, STREAM, MULTI, RESKB>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL); });
        if (e != cudaSuccess) { set_cuda_error(e, "cudaFuncSetAttribute(conv_tc_kernel)"); return B2C_ERR_CUDA; }
    }
    const int sm_count = tc_sm_count();
    int64_t tiles = MULTI ? p.cls_tile0[p.ncls] : (int64_t)((p.M + 127) / 128) * ((p.N + BN - 1) / BN) * splits;
    if (tiles > 0x7fffffffLL) return B2C_ERR_TOO_LARGE;
    TcParams q = p;
    q.splits = splits;
#ifdef B2C_TC_DEV
    { const char* e = getenv("B2C_TC_DBG"); q.dbg = e ? atoi(e) : 0; }
#endif
    int grid = q.sk ? sm_count : (int)(tiles < sm_count ? tiles : sm_count);     // one persistent CTA per SM
    if ((q.stats && q.stats_cta) || RESKB) grid -= grid % ((p.N + BN - 1) / BN);    // a CTA keeps its column tile
    launch_pdl(conv_tc_kernel<MODE, BN, STAGES, SK, SLABS, BSRC, STREAM, MULTI, RESKB>, grid, tc_threads<STREAM>(), L::TOTAL, st, ma, mb0, mb1, mo, ma3 ? *ma3 : ma, q);
    return check_launch("conv_tc_kernel");
}

template <int BSRC>
static int dispatch_fwd(int bn, const CUtensorMap& ma, const CUtensorMap& mb0, const CUtensorMap& mb1, const CUtensorMap& mo, const TcParams& p, cudaStream_t st)
{
    if (p.sk) {
        if (bn == 64) return launch_tc<TCM_FWD, 64, 6, true, 2, BSRC>(ma, mb0, mb1, mo, p, 1, st);
        return launch_tc<TCM_FWD, 128, 4, true, 2, BSRC>(ma, mb0, mb1, mo, p, 1, st);
    }
    // Short K loops are bound by the epilogue.  Tiles of one tensor-memory chunk (at most TC_CHUNK k-blocks) take the
    // streaming epilogue (32 columns at a time straight from tensor memory); up to four k-blocks per tile a shallower
    // operand pipeline also leaves room for four output slabs per drain warp, so a whole tile's stores are in flight.
    if (p.kblocks <= 4 && p.tma_store) {
        if constexpr (BSRC != TCB_SPLIT) {
            // The filter tiles of a column tile are a few tens of KB: they stay in shared memory for the whole launch
            // (a CTA keeps one column tile), the ring holds activations only and runs further ahead.
            const int nt = (p.N + bn - 1) / bn;
            const int64_t tiles = (int64_t)((p.M + 127) / 128) * nt;
            if (tiles >= nt && nt <= tc_sm_count()) {
                if (bn == 64) return launch_tc<TCM_FWD, 64, 6, false, 2, BSRC, TC_STREAM8, false, 4>(ma, mb0, mb1, mo, p, 1, st);
                if (p.kblocks <= 2) return launch_tc<TCM_FWD, 128, 6, false, 2, BSRC, TC_STREAM8, false, 2>(ma, mb0, mb1, mo, p, 1, st);
                return launch_tc<TCM_FWD, 128, 4, false, 1, BSRC, TC_STREAM8, false, 4>(ma, mb0, mb1, mo, p, 1, st);
            }
        }
        if (bn == 64) return launch_tc<TCM_FWD, 64, 4, false, 2, BSRC, TC_STREAM8>(ma, mb0, mb1, mo, p, 1, st);
        return launch_tc<TCM_FWD, 128, 3, false, 2, BSRC, TC_STREAM8>(ma, mb0, mb1, mo, p, 1, st);
    }
    if (p.kblocks <= TC_CHUNK && p.tma_store) {
        if (bn == 64) return launch_tc<TCM_FWD, 64, 6, false, 2, BSRC, 1>(ma, mb0, mb1, mo, p, 1, st);
        return launch_tc<TCM_FWD, 128, 4, false, 2, BSRC, 1>(ma, mb0, mb1, mo, p, 1, st);
    }
    if (bn == 64) return launch_tc<TCM_FWD, 64, 6, false, 2, BSRC>(ma, mb0, mb1, mo, p, 1, st);
    return launch_tc<TCM_FWD, 128, 4, false, 2, BSRC>(ma, mb0, mb1, mo, p, 1, st);
}

static int dispatch_wgrad(int bn, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, const TcParams& p, int splits, cudaStream_t st)
{
    if (bn == 64) return launch_tc<TCM_WGRAD, 64, 6, false, 2, TCB_SPLIT>(ma, mb, mb, mo, p, splits, st);
    return launch_tc<TCM_WGRAD, 128, 4, false, 2, TCB_SPLIT>(ma, mb, mb, mo, p, splits, st);
}

// The caller's filter as a 3-D tensor [d2][d1 = taps][d0 = contiguous channel], box = 32 channels x 1 tap x box2.
static bool make_map_filter(CUtensorMap* map, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
                            uint64_t stride2_bytes, uint32_t box2, CUtensorMapSwizzle swz)
{
    cuuint64_t dims[3] = {d0, d1, d2};
    cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
    cuuint32_t box[3] = {32, 1, box2};
    cuuint32_t estr[3] = {1, 1, 1};
    return g_encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Output seen as [planes][rows][cols] floats, box = 32 cols x 32 rows (x 1 plane), 128B swizzle.
// planes == 0 asks for the 2-D form (the forward kernel stores with 2-D coordinates, the weight-gradient
// kernel always with 3-D ones, so the rank must match the kernel, not the data).
static bool make_map_out(CUtensorMap* map, const void* base, uint64_t planes, uint64_t rows, uint64_t cols)
{
    if (planes == 0) {
        cuuint64_t dims[2] = {cols, rows};
        cuuint64_t strides[1] = {cols * sizeof(float)};
        cuuint32_t box[2] = {32, 32};
        cuuint32_t estr[2] = {1, 1};
        return g_encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    }
    cuuint64_t dims[3] = {cols, rows, planes};
    cuuint64_t strides[2] = {cols * sizeof(float), rows * cols * sizeof(float)};
    cuuint32_t box[3] = {32, 32, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return g_encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// fprop-shaped launch: `act` (n, ah, aw, C) gathered through a window whose first position is
// (low_h, low_w), with cnt_h x cnt_w positions per image and traversal stride (str_h, str_w); virtual
// filter kh x kw (dilation dil); output rows (n, i, j) over P x Q written at out + n*o_sn + i*o_sh + j*o_sw.
// Where a forward pass leaves the batch statistics of its output (see TcParams::stats), or null.
struct StatsOut { float* sums; };

// Whole tiles or balanced k-block ranges for a forward launch (cost in k-block units: whole tiles take
// rounds x kblocks; balanced ranges take units / G plus the hand-over of one partial tile: store, flag, load, add,
// about four k-blocks).
static bool fwd_prefers_balanced(int64_t M, int N, int64_t kblocks)
{
    const int G = tc_sm_count();
    const int BN = N <= 64 ? 64 : 128;
    const int64_t tiles = ((M + 127) / 128) * ((N + BN - 1) / BN);
    const int64_t rounds = (tiles + G - 1) / G;
    const double plain = (double)rounds * (double)kblocks, balanced = (double)(tiles * kblocks) / G + 4.0;
    return tiles * kblocks >= 4 * (int64_t)G && balanced < tc_balance_threshold() * plain;
}

// Rows of the statistics buffer a forward launch with batch sums writes: one per CTA group and row quadrant when the
// launch takes whole tiles (a CTA then keeps its column tile and sums over all its tiles), else one per 32 output rows.
static int64_t fwd_stats_rows(int64_t M, int N, int64_t kblocks, bool may_balance, bool* by_cta)
{
    const int G = tc_sm_count();
    const int BN = N <= 64 ? 64 : 128;
    const int64_t nt = (N + BN - 1) / BN, tiles = ((M + 127) / 128) * nt;
    const int64_t grid = tiles < G ? tiles : G;
    const bool cta = nt <= grid && !(may_balance && fwd_prefers_balanced(M, N, kblocks));
    if (by_cta) *by_cta = cta;
    return cta ? (grid / nt) * 4 : (M + 31) / 32;
}
// Stride-2 data gradient of a 1x1 filter: the launch writes class (0, 0) and the zeros of the other three (TcParams::zfill).
struct ZeroFill { int W, H; int64_t off_w, off_h; };

struct FwdLaunch {
    int n, ah, aw, C, P, Q, N, kh, kw, low_h, low_w, cnt_h, cnt_w, str_h, str_w, dil_h, dil_w;
    int64_t o_sn, o_sh, o_sw;
};

static int run_fwd(const FwdLaunch& f, const void* act, const void* w, const PrepParams& pp, const void* bias,
                   const b2c_bn_params* bn, int relu, float* out, void* ws, size_t ws_bytes, cudaStream_t st,
                   bool filters_ready = false, const StatsOut* stats = nullptr, const ZeroFill* zf = nullptr)
{
    if (!load_driver_entry_points()) return B2C_ERR_UNSUPPORTED;
    const int64_t K = (int64_t)f.kh * f.kw * f.C;
    const size_t fbytes = align_up((size_t)f.N * K * sizeof(float), 1024);
    uintptr_t base = align_up((uintptr_t)ws, 1024);
    if (!ws || base + 2 * fbytes > (uintptr_t)ws + ws_bytes) return B2C_ERR_WORKSPACE_TOO_SMALL;
    if (((uintptr_t)act & 15) || ((uintptr_t)out & 15)) return B2C_ERR_MISALIGNED;
    float* w_hi = (float*)base;
    float* w_lo = (float*)(base + fbytes);
    const int BN = f.N <= 64 ? 64 : 128;
    // Balanced mode when whole tiles would leave a large part of the last round of the CTA grid idle.
    int sk = 0;
    int* sk_flags = (int*)(base + 2 * fbytes);
    float* sk_partial = (float*)((uintptr_t)sk_flags + sk_flag_bytes());
    // hand-over flags: in the library's self-cleaning bank when this stream has one, else cleared in the workspace
    unsigned int* sk_bank = tc_sm_count() * 4 <= TC_SYNC_FLAGS ? tc_sync_bank(st) : nullptr;
    if (sk_bank) sk_flags = (int*)sk_bank;
    {
        const int64_t kblocks = (int64_t)f.kh * f.kw * (f.C / 32);
        const bool room = base + 2 * fbytes + sk_bytes() <= (uintptr_t)ws + ws_bytes;
        if (!filters_ready && room && fwd_prefers_balanced((int64_t)f.n * f.P * f.Q, f.N, kblocks)) sk = 1;
    }
    // The filter itself serves as the B operand when its layout allows a tensor map over it (the channel axis
    // that is contiguous decides K-major or MN-major); otherwise hi/lo copies in the GEMM layout are written first.
    // Splitting the B tile in shared memory costs a long launch about 4 % (measured on a 0.9 ms layer), the split
    // kernel about 5 us: the copies win beyond roughly 125 us of work (0.6 us per k-block on 148 SMs).
    int bsrc = TCB_SPLIT;
    CUtensorMap ma, mbh, mbl;
    const bool long_launch = (((int64_t)f.n * f.P * f.Q + 127) / 128) * ((f.N + BN - 1) / BN) * f.kh * f.kw * (f.C / 32) > 30000;
    if (!filters_ready && !long_launch && ((uintptr_t)w & 15) == 0 && pp.s_r == (int64_t)pp.Sreal * pp.s_s && (pp.s_s * 4) % 16 == 0) {
        const uint64_t taps = (uint64_t)pp.Rreal * pp.Sreal;
        if (pp.s_c == 1 && (pp.s_row * 4) % 16 == 0 &&
            make_map_filter(&mbh, w, (uint64_t)pp.C, taps, (uint64_t)pp.rows, (uint64_t)pp.s_s * 4, (uint64_t)pp.s_row * 4, BN, CU_TENSOR_MAP_SWIZZLE_128B))
            bsrc = TCB_RAW_K;
        else if (pp.s_row == 1 && (pp.s_c * 4) % 16 == 0 &&
                 make_map_filter(&mbh, w, (uint64_t)pp.rows, taps, (uint64_t)pp.C, (uint64_t)pp.s_s * 4, (uint64_t)pp.s_c * 4, 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B))
            bsrc = TCB_RAW_MN;
        if (bsrc != TCB_SPLIT) mbl = mbh;
    }
    if (!filters_ready && bsrc == TCB_SPLIT) {
        int64_t total = (int64_t)f.N * K;
        int blocks = (int)((total + 255) / 256 < tc_sm_count() * 8 ? (total + 255) / 256 : tc_sm_count() * 8);
        launch_pdl(tc_prep_filter_kernel, blocks, 256, 0, st, pp, (const float*)w, w_hi, w_lo, sk_flags, sk && !sk_bank ? tc_sm_count() * 4 : 0);
        int rc = check_launch("tc_prep_filter_kernel");
        if (rc) return rc;
    } else if (sk && !sk_bank) {
        cudaError_t e = cudaMemsetAsync(sk_flags, 0, (size_t)tc_sm_count() * 4 * sizeof(int), st);
        if (e != cudaSuccess) { set_cuda_error(e, "cudaMemsetAsync(balanced-mode flags)"); return B2C_ERR_CUDA; }
    }
    if (!make_map_im2col(&ma, act, f.n, f.ah, f.aw, f.C, f.low_h, f.low_w, f.cnt_h, f.cnt_w, f.str_h, f.str_w, 128)) return B2C_ERR_UNSUPPORTED;
    if (bsrc == TCB_SPLIT && (!make_map_2d(&mbh, w_hi, f.N, K, BN) || !make_map_2d(&mbl, w_lo, f.N, K, BN))) return B2C_ERR_UNSUPPORTED;
    TcParams p{};
    p.M = f.n * f.P * f.Q; p.N = f.N; p.P = f.P; p.Q = f.Q;
    p.C = f.C; p.cblocks = f.C / 32; p.kblocks = f.kh * f.kw * p.cblocks; p.S = f.kw;
    p.str_h = f.str_h; p.str_w = f.str_w; p.dil_h = f.dil_h; p.dil_w = f.dil_w; p.low_h = f.low_h; p.low_w = f.low_w;
    p.bias = (const float*)bias;
    if (bn) { p.mean = (const float*)bn->mean; p.inv_std = (const float*)bn->inv_std; p.gamma = (const float*)bn->gamma; p.beta = (const float*)bn->beta; }
    p.relu = relu;
    p.epi = (p.bias ? TC_EPI_BIAS : 0) | (p.mean ? TC_EPI_BN : 0) | (relu ? TC_EPI_RELU : 0);
    if (f.N % 4 == 0 && !(((uintptr_t)p.bias | (uintptr_t)p.mean | (uintptr_t)p.inv_std | (uintptr_t)p.gamma | (uintptr_t)p.beta) & 15))
        p.epi |= TC_EPI_VEC;
    p.out = out; p.o_sn = f.o_sn; p.o_sh = f.o_sh; p.o_sw = f.o_sw;
    p.tap_r0 = pp.r0; p.tap_rstep = pp.rstep; p.tap_s0 = pp.s0; p.tap_sstep = pp.sstep; p.tap_sreal = pp.Sreal;
    p.sk = sk; p.sk_flags = sk_flags; p.sk_partial = sk_partial; p.sk_selfclean = sk_bank ? 1 : 0;
    // dense rows (plain fprop / stride-1 dgrad): rows are N floats apart in (n, i, j) order
    const bool dense = f.o_sw == f.N && f.o_sh == (int64_t)f.Q * f.N && f.o_sn == (int64_t)f.P * f.Q * f.N;
    CUtensorMap mo = mbh;
    p.tma_store = 0;
    if (dense && make_map_out(&mo, out, 0, (uint64_t)p.M, (uint64_t)f.N)) p.tma_store = 1;
    if (zf) {
        if (p.tma_store || (f.N % 4) || ((zf->off_w | zf->off_h) & 3)) return B2C_ERR_UNSUPPORTED;
        p.zfill = 1; p.z_W = zf->W; p.z_H = zf->H; p.z_w = zf->off_w; p.z_h = zf->off_h;
    }
    if (stats) {
        // the statistics are taken from the staging slabs of the TMA-store epilogue
        if (!p.tma_store) return B2C_ERR_UNSUPPORTED;
        p.stats = stats->sums;
        bool by_cta = false;
        fwd_stats_rows(p.M, p.N, p.kblocks, !filters_ready, &by_cta);
        p.stats_cta = by_cta ? 1 : 0;       // by_cta implies sk == 0: balanced ranges are only taken when preferred
    }
    if (bsrc == TCB_RAW_K) return dispatch_fwd<TCB_RAW_K>(BN, ma, mbh, mbl, mo, p, st);
    if (bsrc == TCB_RAW_MN) return dispatch_fwd<TCB_RAW_MN>(BN, ma, mbh, mbl, mo, p, st);
    return dispatch_fwd<TCB_SPLIT>(BN, ma, mbh, mbl, mo, p, st);
}

static LowerParams lower_params(const Geo& g)
{
    return LowerParams{g.n, g.h, g.w, g.ci, g.ho, g.wo, g.kh, g.kw, g.vpad, g.hpad, g.vstr, g.hstr, g.vdil, g.hdil, (int)g.K, lowered_kp(g)};
}
static int launch_lower(const Geo& g, const void* x, float* rows, cudaStream_t st)
{
    LowerParams lp = lower_params(g);
    const int kq = lp.Kp / 4;
    // one block per output row when its input rows fit in shared memory
    const int wp = (g.wo - 1) * g.hstr + (g.kw - 1) * g.hdil + 1;
    const size_t patch_bytes = (size_t)g.kh * wp * g.ci * sizeof(float);
    if (kq <= 256 && patch_bytes <= 200 * 1024 && (int64_t)g.n * g.ho < 0x7fffffffLL) {
        static PerDeviceOnce attr;
        cudaError_t e = attr.run([] { return cudaFuncSetAttribute(tc_lower_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); });
        if (e != cudaSuccess) { set_cuda_error(e, "cudaFuncSetAttribute(tc_lower_rows_kernel)"); return B2C_ERR_CUDA; }
        const int threads = 256 / kq * kq < 64 ? kq : 256 / kq * kq;       // a whole number of column-group sets
        launch_pdl(tc_lower_rows_kernel, (unsigned)(g.n * g.ho), threads, patch_bytes, st, lp, (const float*)x, (float4*)rows, wp);
        return check_launch("tc_lower_rows_kernel");
    }
    int64_t total = g.M * kq;
    // block count: a multiple of kq / gcd(kq, 256), so that the thread count is a multiple of kq
    int a = kq, b = 256;
    while (b) { int t = a % b; a = b; b = t; }
    const int unit = kq / a;
    int64_t blocks = (total + 255) / 256 < tc_sm_count() * 16 ? (total + 255) / 256 : tc_sm_count() * 16;
    blocks = (blocks + unit - 1) / unit * unit;
    launch_pdl(tc_lower_kernel, (unsigned)blocks, 256, 0, st, lp, (const float*)x, (float4*)rows);
    return check_launch("tc_lower_kernel");
}

static int tc_fprop_nhwc(const Geo& g, const void* x, const void* w, const void* bias, const b2c_bn_params* bn, int relu,
             void* y, void* ws, size_t ws_bytes, cudaStream_t st, const StatsOut* stats = nullptr)
{
    WStride wsd = w_stride(g.w_layout, g.ci, g.co, g.kh, g.kw);
    if (g.ci % 32 != 0) {
        // few-channel layer: write out the im2row matrix, then a 1x1 convolution over it
        const int Kp = lowered_kp(g);
        const size_t lbytes = align_up((size_t)g.M * Kp * sizeof(float), 1024);
        const size_t fbytes = align_up((size_t)g.co * Kp * sizeof(float), 1024);
        uintptr_t base = align_up((uintptr_t)ws, 1024);
        if (!ws || base + lbytes + 2 * fbytes + 1024 > (uintptr_t)ws + ws_bytes) return B2C_ERR_WORKSPACE_TOO_SMALL;
        float* rows = (float*)base;
        float* w_hi = (float*)align_up(base + lbytes, 1024);
        float* w_lo = (float*)((uintptr_t)w_hi + fbytes);
        int rc = launch_lower(g, x, rows, st);
        if (rc) return rc;
        int64_t total = (int64_t)g.co * Kp;
        launch_pdl(tc_prep_filter_lowered_kernel, (int)((total + 255) / 256), 256, 0, st, g.co, (int)g.K, Kp, g.ci, g.kw, wsd.sk, wsd.sc, wsd.sr,
                                                                                 wsd.ss, (const float*)w, w_hi, w_lo);
        rc = check_launch("tc_prep_filter_lowered_kernel");
        if (rc) return rc;
        PrepParams none{};
        FwdLaunch f{g.n, g.ho, g.wo, Kp, g.ho, g.wo, g.co, 1, 1, 0, 0, g.ho, g.wo, 1, 1, 1, 1,
                    (int64_t)g.ho * g.wo * g.co, (int64_t)g.wo * g.co, (int64_t)g.co};
        return run_fwd(f, rows, nullptr, none, bias, bn, relu, (float*)y, (void*)w_hi, 2 * fbytes + 1024, st, true, stats);
    }
    PrepParams pp{g.co, g.ci, g.kh, g.kw, wsd.sk, wsd.sc, wsd.sr, wsd.ss, 0, 1, 0, 1, g.kh, g.kw};
    FwdLaunch f{g.n, g.h, g.w, g.ci, g.ho, g.wo, g.co, g.kh, g.kw, -g.vpad, -g.hpad,
                g.h + 2 * g.vpad - (g.kh - 1) * g.vdil, g.w + 2 * g.hpad - (g.kw - 1) * g.hdil,
                g.vstr, g.hstr, g.vdil, g.hdil, (int64_t)g.ho * g.wo * g.co, (int64_t)g.wo * g.co, (int64_t)g.co};
    return run_fwd(f, x, w, pp, bias, bn, relu, (float*)y, ws, ws_bytes, st, false, stats);
}

// Strided data gradient, all parity classes in one launch (MULTI kernel variants): up to four classes, every class
// with at least one tap, filters read in place.  The tiles of the classes with the most taps come first in the tile
// list, so the persistent CTAs end with the short ones.  Returns 1 when the shape does not qualify.
static int tc_dgrad_classes_one_launch(const Geo& g, const WStride& wsd, const void* dy, const void* w, void* dx, cudaStream_t st)
{
    if (g.vstr * g.hstr > 4 || !load_driver_entry_points()) return 1;
    struct Cls { AxisClass a, b; int ia, ib; };
    Cls cls[4];
    int ncls = 0;
    for (int a = 0; a < g.vstr; a++)
        for (int b = 0; b < g.hstr; b++) {
            AxisClass ca = axis_class(a, g.vstr, g.vpad, g.kh, g.h), cb = axis_class(b, g.hstr, g.hpad, g.kw, g.w);
            if (ca.out_cnt == 0 || cb.out_cnt == 0) continue;
            // A class no tap reaches is all zeros.  Writing them from tiles without k-blocks was tried and is slower
            // than clearing dx with a memset first (the drain warps' staged stores against a copy-engine fill:
            // 119 against 107 us on a 56x56x256 -> 512 1x1 stride-2 layer), so such shapes take the path below.
            if (ca.cnt == 0 || cb.cnt == 0) return 1;
            cls[ncls++] = Cls{ca, cb, a, b};
        }
    if (ncls < 2) return 1;
    for (int i = 0; i < ncls; i++)                              // most taps first
        for (int j = i + 1; j < ncls; j++)
            if (cls[j].a.cnt * cls[j].b.cnt > cls[i].a.cnt * cls[i].b.cnt) { Cls t = cls[i]; cls[i] = cls[j]; cls[j] = t; }
    if (((uintptr_t)dy & 15) || ((uintptr_t)dx & 15) || ((uintptr_t)w & 15)) return 1;
    // the filter as the B operand, in place (see run_fwd): rows = ci (GEMM N), contraction channel = co
    const int64_t s_row = wsd.sc, s_c = wsd.sk, s_r = wsd.sr, s_s = wsd.ss;
    if (s_r != (int64_t)g.kw * s_s || (s_s * 4) % 16) return 1;
    const int BN = g.ci <= 64 ? 64 : 128;
    const uint64_t taps = (uint64_t)g.kh * g.kw;
    CUtensorMap mb;
    int bsrc;
    if (s_c == 1 && (s_row * 4) % 16 == 0 &&
        make_map_filter(&mb, w, (uint64_t)g.co, taps, (uint64_t)g.ci, (uint64_t)s_s * 4, (uint64_t)s_row * 4, BN, CU_TENSOR_MAP_SWIZZLE_128B))
        bsrc = TCB_RAW_K;
    else if (s_row == 1 && (s_c * 4) % 16 == 0 &&
             make_map_filter(&mb, w, (uint64_t)g.ci, taps, (uint64_t)g.co, (uint64_t)s_s * 4, (uint64_t)s_c * 4, 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B))
        bsrc = TCB_RAW_MN;
    else return 1;
    TcParams p{};
    CUtensorMap ma[4];
    const int nt = (g.ci + BN - 1) / BN;
    p.N = g.ci; p.C = g.co; p.cblocks = g.co / 32;
    p.str_h = 1; p.str_w = 1; p.dil_h = 1; p.dil_w = 1;
    p.out = (float*)dx; p.o_sn = (int64_t)g.h * g.w * g.ci; p.o_sh = (int64_t)g.vstr * g.w * g.ci; p.o_sw = (int64_t)g.hstr * g.ci;
    p.tap_rstep = -g.vstr; p.tap_sstep = -g.hstr; p.tap_sreal = g.kw;
    p.splits = 1; p.ncls = ncls;
    int64_t tiles = 0;
    for (int i = 0; i < ncls; i++) {
        const AxisClass &ca = cls[i].a, &cb = cls[i].b;
        if (!make_map_im2col(&ma[i], dy, g.n, g.ho, g.wo, g.co, ca.dmin, cb.dmin, ca.out_cnt, cb.out_cnt, 1, 1, 128)) return 1;
        p.cls_tile0[i] = (int)tiles;
        p.cls_M[i] = g.n * ca.out_cnt * cb.out_cnt; p.cls_P[i] = ca.out_cnt; p.cls_Q[i] = cb.out_cnt;
        p.cls_kblocks[i] = ca.cnt * cb.cnt * p.cblocks; p.cls_S[i] = cb.cnt;
        p.cls_low_h[i] = ca.dmin; p.cls_low_w[i] = cb.dmin; p.cls_r0[i] = ca.r0; p.cls_s0[i] = cb.r0;
        p.cls_out[i] = ((int64_t)cls[i].ia * g.w + cls[i].ib) * g.ci;
        tiles += (int64_t)((p.cls_M[i] + 127) / 128) * nt;
        if (tiles > 0x7fffffffLL) return 1;
    }
    for (int i = ncls; i < 4; i++) ma[i] = ma[0];
    p.cls_tile0[ncls] = (int)tiles;
    // launch-wide fields the kernel still reads
    p.M = p.cls_M[0]; p.P = p.cls_P[0]; p.Q = p.cls_Q[0]; p.kblocks = p.cls_kblocks[0]; p.S = p.cls_S[0];
    if (bsrc == TCB_RAW_K) {
        if (BN == 64) return launch_tc<TCM_FWD, 64, 6, false, 2, TCB_RAW_K, 0, true>(ma[0], mb, ma[1], ma[2], p, 1, st, &ma[3]);
        return launch_tc<TCM_FWD, 128, 4, false, 2, TCB_RAW_K, 0, true>(ma[0], mb, ma[1], ma[2], p, 1, st, &ma[3]);
    }
    if (BN == 64) return launch_tc<TCM_FWD, 64, 6, false, 2, TCB_RAW_MN, 0, true>(ma[0], mb, ma[1], ma[2], p, 1, st, &ma[3]);
    return launch_tc<TCM_FWD, 128, 4, false, 2, TCB_RAW_MN, 0, true>(ma[0], mb, ma[1], ma[2], p, 1, st, &ma[3]);
}

static int tc_dgrad_nhwc(const Geo& g, const void* dy, const void* w, void* dx, void* ws, size_t ws_bytes, cudaStream_t st)
{
    WStride wsd = w_stride(g.w_layout, g.ci, g.co, g.kh, g.kw);
    if (g.vstr == 1 && g.hstr == 1) {
        // dx = convolution of dy with the flipped, transposed filter and padding (k-1)*dil - pad
        const int pv = (g.kh - 1) * g.vdil - g.vpad, ph = (g.kw - 1) * g.hdil - g.hpad;
        PrepParams pp{g.ci, g.co, g.kh, g.kw, wsd.sc, wsd.sk, wsd.sr, wsd.ss, g.kh - 1, -1, g.kw - 1, -1, g.kh, g.kw};
        FwdLaunch f{g.n, g.ho, g.wo, g.co, g.h, g.w, g.ci, g.kh, g.kw, -pv, -ph, g.h, g.w, 1, 1, g.vdil, g.hdil,
                    (int64_t)g.h * g.w * g.ci, (int64_t)g.w * g.ci, (int64_t)g.ci};
        return run_fwd(f, dy, w, pp, nullptr, nullptr, 0, (float*)dx, ws, ws_bytes, st);
    }
    // Strided: the input positions split into str_h*str_w parity classes; each class is a dense
    // stride-1 convolution of dy with the sub-filter of the taps that reach it, written to its
    // strided positions of dx. Classes no tap reaches stay zero.
    {
        int rc = tc_dgrad_classes_one_launch(g, wsd, dy, w, dx, st);
        if (rc != 1) return rc;            // 1: not applicable, one launch per class below
    }
    bool any_empty = false;
    int live = 0;
    for (int a = 0; a < g.vstr; a++)
        for (int b = 0; b < g.hstr; b++) {
            AxisClass ca = axis_class(a, g.vstr, g.vpad, g.kh, g.h), cb = axis_class(b, g.hstr, g.hpad, g.kw, g.w);
            if ((ca.cnt == 0 || cb.cnt == 0) && ca.out_cnt > 0 && cb.out_cnt > 0) any_empty = true;
            if (ca.cnt > 0 && cb.cnt > 0 && ca.out_cnt > 0 && cb.out_cnt > 0) live++;
        }
    {
        // 2 x 2 stride, only class (0, 0) reached by a tap (a 1x1 filter without padding): the class's launch writes the
        // other classes' zeros next to its own rows, no clearing pass over dx
        AxisClass ca = axis_class(0, g.vstr, g.vpad, g.kh, g.h), cb = axis_class(0, g.hstr, g.hpad, g.kw, g.w);
        if (g.vstr == 2 && g.hstr == 2 && live == 1 && ca.cnt > 0 && cb.cnt > 0 && g.ci % 4 == 0 && ((uintptr_t)dx & 15) == 0) {
            PrepParams pp{g.ci, g.co, ca.cnt, cb.cnt, wsd.sc, wsd.sk, wsd.sr, wsd.ss, ca.r0, -g.vstr, cb.r0, -g.hstr, g.kh, g.kw};
            FwdLaunch f{g.n, g.ho, g.wo, g.co, ca.out_cnt, cb.out_cnt, g.ci, ca.cnt, cb.cnt, ca.dmin, cb.dmin,
                        ca.out_cnt, cb.out_cnt, 1, 1, 1, 1,
                        (int64_t)g.h * g.w * g.ci, (int64_t)g.vstr * g.w * g.ci, (int64_t)g.hstr * g.ci};
            ZeroFill zf{g.w, g.h, (int64_t)g.ci, (int64_t)g.w * g.ci};
            int rc = run_fwd(f, dy, w, pp, nullptr, nullptr, 0, (float*)dx, ws, ws_bytes, st, false, nullptr, &zf);
            if (rc != B2C_ERR_UNSUPPORTED) return rc;
        }
    }
    if (any_empty) {
        cudaError_t e = cudaMemsetAsync(dx, 0, (size_t)g.n * g.h * g.w * g.ci * sizeof(float), st);
        if (e != cudaSuccess) { set_cuda_error(e, "cudaMemsetAsync(dx)"); return B2C_ERR_CUDA; }
    }
    for (int a = 0; a < g.vstr; a++)
        for (int b = 0; b < g.hstr; b++) {
            AxisClass ca = axis_class(a, g.vstr, g.vpad, g.kh, g.h), cb = axis_class(b, g.hstr, g.hpad, g.kw, g.w);
            if (ca.out_cnt == 0 || cb.out_cnt == 0 || ca.cnt == 0 || cb.cnt == 0) continue;
            PrepParams pp{g.ci, g.co, ca.cnt, cb.cnt, wsd.sc, wsd.sk, wsd.sr, wsd.ss, ca.r0, -g.vstr, cb.r0, -g.hstr, g.kh, g.kw};
            FwdLaunch f{g.n, g.ho, g.wo, g.co, ca.out_cnt, cb.out_cnt, g.ci, ca.cnt, cb.cnt, ca.dmin, cb.dmin,
                        ca.out_cnt, cb.out_cnt, 1, 1, 1, 1,
                        (int64_t)g.h * g.w * g.ci, (int64_t)g.vstr * g.w * g.ci, (int64_t)g.hstr * g.ci};
            float* out = (float*)dx + ((int64_t)a * g.w + b) * g.ci;
            int rc = run_fwd(f, dy, w, pp, nullptr, nullptr, 0, out, ws, ws_bytes, st);
            if (rc) return rc;
        }
    return B2C_OK;
}

static int tc_wgrad_nhwc(const Geo& g, const void* x, const void* dy, void* dw, void* db, void* ws, size_t ws_bytes, cudaStream_t st,
                         bool lowered_in_ws = false, bool exchanged = false)
{
    if (!load_driver_entry_points()) return B2C_ERR_UNSUPPORTED;
    if (!exchanged && !db && !lowered_in_ws && wgrad_swap_ok(g))
        return tc_wgrad_nhwc(wgrad_swapped(g), dy, x, dw, nullptr, ws, ws_bytes, st, false, true);
    const bool low = g.ci % 32 != 0;
    const int Krows = low ? lowered_kp(g) : (int)g.K;
    WgradPlan pl = wgrad_plan(g);
    const size_t lbytes = low ? align_up((size_t)g.M * Krows * sizeof(float), 1024) : 0;
    const size_t pbytes = align_up((size_t)pl.splits * Krows * g.co * sizeof(float), 1024);
    uintptr_t base = align_up((uintptr_t)ws, 1024);
    const size_t cs = align_up((size_t)pl.splits * 4 * g.co * sizeof(float), 1024);
    if (!ws || base + lbytes + pbytes + (db ? cs : 0) > (uintptr_t)ws + ws_bytes) return B2C_ERR_WORKSPACE_TOO_SMALL;
    if (((uintptr_t)x & 15) || ((uintptr_t)dy & 15)) return B2C_ERR_MISALIGNED;
    float* partial = (float*)(base + lbytes);
    CUtensorMap ma, mb;
    TcParams p{};
    if (low) {
        // few-channel layer: gradient of the 1x1 convolution over the written-out im2row matrix
        float* rows = (float*)base;
        if (!lowered_in_ws) {               // else: the forward pass of this layer left the matrix here (same offset)
            int rc = launch_lower(g, x, rows, st);
            if (rc) return rc;
        }
        int lg = Krows % 128 == 0 ? 7 : Krows % 64 == 0 ? 6 : 5;       // widest box first, narrower if the encoder refuses
        while (lg >= 5 && !make_map_im2col(&ma, rows, g.n, g.ho, g.wo, Krows, 0, 0, g.ho, g.wo, 1, 1, 32, CU_TENSOR_MAP_SWIZZLE_NONE, 1u << lg)) lg--;
        if (lg < 5) return B2C_ERR_UNSUPPORTED;
        p.a_box_log2 = lg;
        p.C = Krows; p.cblocks = Krows / 32; p.S = 1;
        p.str_h = 1; p.str_w = 1; p.dil_h = 1; p.dil_w = 1; p.low_h = 0; p.low_w = 0;
    } else {
        // x boxes as wide as the channel count allows (fewer TMA instructions per k-block: the producer's issue
        // time was 36-63 % of the kernel's on the weight gradients of the step)
        int lg = g.ci % 128 == 0 ? 7 : g.ci % 64 == 0 ? 6 : 5;
        while (lg >= 5 && !make_map_im2col(&ma, x, g.n, g.h, g.w, g.ci, -g.vpad, -g.hpad, g.h + 2 * g.vpad - (g.kh - 1) * g.vdil,
                                           g.w + 2 * g.hpad - (g.kw - 1) * g.hdil, g.vstr, g.hstr, 32, CU_TENSOR_MAP_SWIZZLE_NONE, 1u << lg)) lg--;
        if (lg < 5) return B2C_ERR_UNSUPPORTED;
        p.a_box_log2 = lg;
        p.C = g.ci; p.cblocks = g.ci / 32; p.S = g.kw;
        p.str_h = g.vstr; p.str_w = g.hstr; p.dil_h = g.vdil; p.dil_w = g.hdil; p.low_h = -g.vpad; p.low_w = -g.hpad;
    }
    if (!make_map_2d(&mb, dy, (uint64_t)g.M, (uint64_t)g.co, 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)) return B2C_ERR_UNSUPPORTED;
    p.M = Krows; p.N = g.co; p.P = g.ho; p.Q = g.wo; p.kblocks = pl.kblocks;
    p.Mpix = (int)g.M;
    p.out = partial;
    p.db_partial = db ? (float*)(base + lbytes + pbytes) : nullptr;
    CUtensorMap mo = mb;
    p.tma_store = make_map_out(&mo, partial, (uint64_t)pl.splits, (uint64_t)Krows, (uint64_t)g.co) ? 1 : 0;
    WStride wsd = w_stride(g.w_layout, g.ci, g.co, g.kh, g.kw);
    if (exchanged) {
        // g is the layer with ci and co exchanged: the caller's filter has g.co input and g.ci output channels
        wsd = w_stride(g.w_layout, g.co, g.ci, 1, 1);
        const int64_t t = wsd.sk; wsd.sk = wsd.sc; wsd.sc = t;
    }
    int rc = dispatch_wgrad(pl.bn, ma, mb, mo, p, pl.splits, st);
    if (rc) return rc;
    WgradReduceParams rp{Krows, g.co, g.ci, g.kw, pl.splits, wsd.sk, wsd.sc, wsd.sr, wsd.ss, (int)g.K};
    if ((int64_t)((g.co + 31) / 32) * ((Krows + 31) / 32) >= 2 * (int64_t)tc_sm_count())
        launch_pdl(tc_wgrad_reduce_kernel<4>, dim3((g.co + 31) / 32, (Krows + 31) / 32), dim3(32, 8), 0, st, rp, partial, (float*)dw, p.db_partial, (float*)db);
    else if ((int64_t)((g.co + 31) / 32) * ((Krows + 7) / 8) >= 2 * (int64_t)tc_sm_count() || pl.splits < 16)
        launch_pdl(tc_wgrad_reduce_kernel<1>, dim3((g.co + 31) / 32, (Krows + 7) / 8), dim3(32, 8), 0, st, rp, partial, (float*)dw, p.db_partial, (float*)db);
    else
        launch_pdl(tc_wgrad_reduce_deep_kernel, dim3((g.co + 31) / 32, Krows), dim3(32, 8), 0, st, rp, partial, (float*)dw, p.db_partial, (float*)db);
    return check_launch("tc_wgrad_reduce_kernel");
}

// ---------------------------------------------------------------------------------------------
// NCHW float32: the same kernels on channel-last copies.  The activations are transposed into the workspace
// (and the result back), as the reference's own NCHW path transposes around its GEMM
// (pydtnn/backends/cpu/layers/conv_2d_cpu.py:264-291, 447-481); filters stay where they are (every filter layout
// is read through strides).  Taken when the transposes cost less than the FMA engine would lose.
// ---------------------------------------------------------------------------------------------
// src [n][rows][cols] -> dst [n][cols][rows]; block (32, 8), grid (cols/32, rows/32, n)
__global__ void transpose_inner_kernel(const float* __restrict__ src, float* __restrict__ dst, int rows, int cols)
{
    pdl_prologue();
    __shared__ float tile[32][33];
    const int64_t plane = (int64_t)rows * cols;
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32, tx = threadIdx.x, ty = threadIdx.y;
    {
        const int img = blockIdx.z;
        const float* s = src + img * plane;
        float* d = dst + img * plane;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int r = r0 + ty + 8 * j, c = c0 + tx;
            if (r < rows && c < cols) tile[ty + 8 * j][tx] = s[(int64_t)r * cols + c];
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int c = c0 + ty + 8 * j, r = r0 + tx;
            if (r < rows && c < cols) d[(int64_t)c * rows + r] = tile[tx][ty + 8 * j];
        }
    }
}

// The same transpose when one extent is at most 8 (the three channels of a network's input): a 32 x 32 tile would
// leave nine tenths of its threads idle.  One thread per position of the long axis; ROWS_THIN: src [n][thin][len]
// -> dst [n][len][thin], else src [n][len][thin] -> dst [n][thin][len].  Loads or stores of a warp cover whole
// contiguous runs either way.
template <bool ROWS_THIN>
__global__ void __launch_bounds__(256) transpose_thin_kernel(const float* __restrict__ src, float* __restrict__ dst, int thin, int len)
{
    pdl_prologue();
    const int l = blockIdx.x * blockDim.x + threadIdx.x;
    if (l >= len) return;
    const int64_t plane = (int64_t)thin * len;
    const float* s = src + blockIdx.y * plane;
    float* d = dst + blockIdx.y * plane;
    float v[8];
#pragma unroll
    for (int r = 0; r < 8; r++)
        if (r < thin) v[r] = ROWS_THIN ? s[(int64_t)r * len + l] : s[(int64_t)l * thin + r];
#pragma unroll
    for (int r = 0; r < 8; r++)
        if (r < thin) { if (ROWS_THIN) d[(int64_t)l * thin + r] = v[r]; else d[(int64_t)r * len + l] = v[r]; }
}

static int transpose_inner(const void* src, void* dst, int n, int rows, int cols, cudaStream_t st)
{
    if (n > 65535) return B2C_ERR_TOO_LARGE;
    if (rows <= 8 && cols > 8) {
        launch_pdl(transpose_thin_kernel<true>, dim3((cols + 255) / 256, n), 256, 0, st, (const float*)src, (float*)dst, rows, cols);
        return check_launch("transpose_thin_kernel");
    }
    if (cols <= 8 && rows > 8) {
        launch_pdl(transpose_thin_kernel<false>, dim3((rows + 255) / 256, n), 256, 0, st, (const float*)src, (float*)dst, cols, rows);
        return check_launch("transpose_thin_kernel");
    }
    launch_pdl(transpose_inner_kernel, dim3((cols + 31) / 32, (rows + 31) / 32, n), dim3(32, 8), 0, st,
               (const float*)src, (float*)dst, rows, cols);
    return check_launch("transpose_inner_kernel");
}

static Geo as_nhwc(const Geo& g) { Geo q = g; q.layout = B2C_LAYOUT_NHWC; return q; }
static size_t act_bytes(int64_t n, int64_t h, int64_t w, int64_t c) { return align_up((size_t)(n * h * w * c) * sizeof(float), 1024); }

bool tc_supported(const Geo& g, int pass)
{
    if (g.layout == B2C_LAYOUT_NHWC) return tc_supported_nhwc(g, pass);
    if (g.dtype != B2C_F32 || g.engine == B2C_ENGINE_FMA || g.n > 65535) return false;
    const Geo q = as_nhwc(g);
    if (!tc_supported_nhwc(q, pass)) return false;
    if (g.engine == B2C_ENGINE_TENSOR) return true;
    // two tensors are copied there and/or back (read + write each) at about 2.5 TB/s; the FMA engine runs the
    // pass at about 26 TFLOP/s, this engine at about 130
    const double flops = 2.0 * (double)g.M * (double)g.K * g.co;
    const double xb = 4.0 * g.n * g.h * g.w * g.ci, yb = 4.0 * (double)g.M * g.co;
    const double moved = 2.0 * (xb + yb);
    return flops / 130e12 + moved / 2.5e12 < flops / 26e12;
}

size_t tc_workspace_bytes(const Geo& g, int pass)
{
    if (g.layout == B2C_LAYOUT_NHWC) return tc_workspace_bytes_nhwc(g, pass);
    return act_bytes(g.n, g.h, g.w, g.ci) + act_bytes(g.n, g.ho, g.wo, g.co) + 1024 + tc_workspace_bytes_nhwc(as_nhwc(g), pass);
}

// workspace of an NCHW call: [x or dx, channel-last][y or dy, channel-last][workspace of the channel-last pass]
struct NchwWs { float *a, *b; void* inner; size_t inner_bytes; };
static bool nchw_ws(const Geo& g, void* ws, size_t ws_bytes, NchwWs& o)
{
    if (!ws) return false;
    const uintptr_t base = align_up((uintptr_t)ws, 1024);
    const size_t xa = act_bytes(g.n, g.h, g.w, g.ci), ya = act_bytes(g.n, g.ho, g.wo, g.co);
    if (base + xa + ya > (uintptr_t)ws + ws_bytes) return false;
    o.a = (float*)base; o.b = (float*)(base + xa); o.inner = (void*)(base + xa + ya);
    o.inner_bytes = (uintptr_t)ws + ws_bytes - (base + xa + ya);
    return true;
}

// Forward pass that also leaves the per-channel sums of its output for a training-mode batch norm (NHWC float32 on this
// engine only).  Buffer: [rows][2][co] floats, rows as fwd_stats_rows says.
size_t tc_stats_bytes(const Geo& g)
{
    if (g.layout != B2C_LAYOUT_NHWC || !tc_supported_nhwc(g, B2C_PASS_FPROP) || g.co % 4) return 0;
    const bool lowered = g.ci % 32 != 0;        // few-channel layers run as a 1x1 convolution over the lowered matrix
    const int64_t kblocks = lowered ? lowered_kp(g) / 32 : (int64_t)g.kh * g.kw * (g.ci / 32);
    return (size_t)fwd_stats_rows(g.M, g.co, kblocks, !lowered, nullptr) * 2 * g.co * sizeof(float);
}

int tc_fprop_stats(const Geo& g, const void* x, const void* w, const void* bias, void* y, void* stats, size_t stats_bytes,
                   void* ws, size_t ws_bytes, cudaStream_t st)
{
    const size_t need = tc_stats_bytes(g);
    if (!need) return B2C_ERR_UNSUPPORTED;
    if (stats_bytes < need) return B2C_ERR_WORKSPACE_TOO_SMALL;
    if ((uintptr_t)stats & 15) return B2C_ERR_MISALIGNED;
    StatsOut so{(float*)stats};
    return tc_fprop_nhwc(g, x, w, bias, nullptr, 0, y, ws, ws_bytes, st, &so);
}

int tc_fprop(const Geo& g, const void* x, const void* w, const void* bias, const b2c_bn_params* bn, int relu,
             void* y, void* ws, size_t ws_bytes, cudaStream_t st)
{
    if (g.layout == B2C_LAYOUT_NHWC) return tc_fprop_nhwc(g, x, w, bias, bn, relu, y, ws, ws_bytes, st);
    NchwWs t;
    if (!nchw_ws(g, ws, ws_bytes, t)) return B2C_ERR_WORKSPACE_TOO_SMALL;
    int rc = transpose_inner(x, t.a, g.n, g.ci, g.h * g.w, st);                 // (c, hw) -> (hw, c)
    if (rc) return rc;
    rc = tc_fprop_nhwc(as_nhwc(g), t.a, w, bias, bn, relu, t.b, t.inner, t.inner_bytes, st);
    if (rc) return rc;
    return transpose_inner(t.b, y, g.n, g.ho * g.wo, g.co, st);                 // (hw, c) -> (c, hw)
}

int tc_dgrad(const Geo& g, const void* dy, const void* w, void* dx, void* ws, size_t ws_bytes, cudaStream_t st)
{
    if (g.layout == B2C_LAYOUT_NHWC) return tc_dgrad_nhwc(g, dy, w, dx, ws, ws_bytes, st);
    NchwWs t;
    if (!nchw_ws(g, ws, ws_bytes, t)) return B2C_ERR_WORKSPACE_TOO_SMALL;
    int rc = transpose_inner(dy, t.b, g.n, g.co, g.ho * g.wo, st);
    if (rc) return rc;
    rc = tc_dgrad_nhwc(as_nhwc(g), t.b, w, t.a, t.inner, t.inner_bytes, st);
    if (rc) return rc;
    return transpose_inner(t.a, dx, g.n, g.h * g.w, g.ci, st);
}

// Few-channel NHWC layers write the im2row matrix of x at the start of the workspace in their forward pass and again
// in their weight gradient.  A caller that gives the layer a workspace of its own can say that the forward pass's
// matrix is still there.
bool tc_keeps_lowered(const Geo& g) { return g.layout == B2C_LAYOUT_NHWC && g.ci % 32 != 0 && tc_supported_nhwc(g, B2C_PASS_WGRAD) && tc_supported_nhwc(g, B2C_PASS_FPROP); }
int tc_wgrad_lowered(const Geo& g, const void* x, const void* dy, void* dw, void* db, void* ws, size_t ws_bytes, cudaStream_t st)
{
    if (!tc_keeps_lowered(g)) return B2C_ERR_UNSUPPORTED;
    return tc_wgrad_nhwc(g, x, dy, dw, db, ws, ws_bytes, st, true);
}

int tc_wgrad(const Geo& g, const void* x, const void* dy, void* dw, void* db, void* ws, size_t ws_bytes, cudaStream_t st)
{
    if (g.layout == B2C_LAYOUT_NHWC) return tc_wgrad_nhwc(g, x, dy, dw, db, ws, ws_bytes, st);
    NchwWs t;
    if (!nchw_ws(g, ws, ws_bytes, t)) return B2C_ERR_WORKSPACE_TOO_SMALL;
    int rc = transpose_inner(x, t.a, g.n, g.ci, g.h * g.w, st);
    if (rc) return rc;
    rc = transpose_inner(dy, t.b, g.n, g.co, g.ho * g.wo, st);
    if (rc) return rc;
    return tc_wgrad_nhwc(as_nhwc(g), t.a, t.b, dw, db, t.inner, t.inner_bytes, st);
}

// ---------------------------------------------------------------------------------------------
// Fully connected layers with a small batch (pydtnn/backends/gpu/layers/fc_gpu.py:54-94: y = x w + b, dw = x^T dy,
// dx = dy w^T, w stored (in, out))
// ---------------------------------------------------------------------------------------------
// With 32-128 rows in x every pass is a stream over the (in, out) weight matrix.  As a 1x1 convolution over `batch`
// pixels the batch is the GEMM row axis and fills a fraction of each 128-row MMA; here the weight matrix takes that
// axis instead: it is read as an activation tensor of `in` pixels with `out` channels, and the batch becomes the
// narrow column axis.
//   forward   y (batch, out)  = weight-gradient form: "x" = w (in pixels x out channels), "dy" = x^T (in x batch),
//                               result in (co = batch, ci = out) filter layout = y; then the bias.
//   dx        dx^T (in, batch) = forward form over w with dy (batch, out) as the (co, ci) filter; then transposed.
//   dw        dw (in, out)    = forward form over x^T (in pixels x batch channels) with dy as the (ci, co) filter.
// x^T and dx^T are batch x in floats: small copies beside one pass over the weights.
static Geo fc_pixels_view(int pixels, int ci, int co, int w_layout)
{
    Geo q{};
    q.layout = B2C_LAYOUT_NHWC; q.dtype = B2C_F32; q.w_layout = w_layout; q.engine = B2C_ENGINE_TENSOR;
    q.n = 1; q.h = pixels; q.w = 1; q.ci = ci; q.co = co; q.kh = q.kw = 1;
    q.vstr = q.hstr = q.vdil = q.hdil = 1;
    q.ho = pixels; q.wo = 1; q.M = pixels; q.K = ci;
    return q;
}

bool tc_fc_small_batch(int dtype, int engine, int batch, int in_f, int out_f)
{
    if (dtype != B2C_F32 || engine == B2C_ENGINE_FMA) return false;
    if (batch > 128 || batch % 32 || out_f % 32 || in_f % 4) return false;
    return (int64_t)in_f * out_f >= (1 << 22);          // a weight matrix of at least 16 MB
}

__global__ void fc_add_bias_kernel(float4* __restrict__ y, const float4* __restrict__ bias, int rows, int cols4)
{
    pdl_prologue();
    const int64_t total = (int64_t)rows * cols4;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        float4 v = y[i];
        const float4 b = bias[i % cols4];
        v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
        y[i] = v;
    }
}

size_t tc_fc_small_batch_bytes(int batch, int in_f, int out_f)
{
    const size_t copy = act_bytes(1, in_f, 1, batch);               // x^T or dx^T
    size_t inner = tc_workspace_bytes_nhwc(fc_pixels_view(in_f, out_f, batch, B2C_W_KRSC), B2C_PASS_WGRAD);
    size_t b = tc_workspace_bytes_nhwc(fc_pixels_view(in_f, out_f, batch, B2C_W_KRSC), B2C_PASS_FPROP);
    if (b > inner) inner = b;
    b = tc_workspace_bytes_nhwc(fc_pixels_view(in_f, batch, out_f, B2C_W_CRSK), B2C_PASS_FPROP);
    if (b > inner) inner = b;
    b = channel_sum_workspace_bytes(batch, out_f, 1);
    if (b > inner) inner = b;
    return copy + inner + 2048;
}

// Splits the caller's workspace into the transposed copy and the rest.
static bool fc_ws(int batch, int in_f, void* ws, size_t ws_bytes, float** copy, void** inner, size_t* inner_bytes)
{
    if (!ws) return false;
    const uintptr_t base = align_up((uintptr_t)ws, 1024);
    const size_t cb = act_bytes(1, in_f, 1, batch);
    if (base + cb > (uintptr_t)ws + ws_bytes) return false;
    *copy = (float*)base; *inner = (void*)(base + cb); *inner_bytes = (uintptr_t)ws + ws_bytes - (base + cb);
    return true;
}

int tc_fc_forward_small_batch(int batch, int in_f, int out_f, const void* x, const void* w, const void* bias, void* y,
                              void* ws, size_t ws_bytes, cudaStream_t st)
{
    float* xt; void* inner; size_t inner_bytes;
    if (!fc_ws(batch, in_f, ws, ws_bytes, &xt, &inner, &inner_bytes)) return B2C_ERR_WORKSPACE_TOO_SMALL;
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y | (uintptr_t)bias) & 15) return B2C_ERR_MISALIGNED;
    int rc = transpose_inner(x, xt, 1, batch, in_f, st);                        // (batch, in) -> (in, batch)
    if (rc) return rc;
    rc = tc_wgrad_nhwc(fc_pixels_view(in_f, out_f, batch, B2C_W_KRSC), w, xt, y, nullptr, inner, inner_bytes, st);
    if (rc || !bias) return rc;
    const int64_t total4 = (int64_t)batch * out_f / 4;
    launch_pdl(fc_add_bias_kernel, (int)((total4 + 255) / 256 < 1184 ? (total4 + 255) / 256 : 1184), 256, 0, st, (float4*)y, (const float4*)bias, batch, out_f / 4);
    return check_launch("fc_add_bias_kernel");
}

int tc_fc_dgrad_small_batch(int batch, int in_f, int out_f, const void* dy, const void* w, void* dx, void* ws, size_t ws_bytes, cudaStream_t st)
{
    float* dxt; void* inner; size_t inner_bytes;
    if (!fc_ws(batch, in_f, ws, ws_bytes, &dxt, &inner, &inner_bytes)) return B2C_ERR_WORKSPACE_TOO_SMALL;
    if (((uintptr_t)dy | (uintptr_t)w | (uintptr_t)dx) & 15) return B2C_ERR_MISALIGNED;
    int rc = tc_fprop_nhwc(fc_pixels_view(in_f, out_f, batch, B2C_W_KRSC), w, dy, nullptr, nullptr, 0, dxt, inner, inner_bytes, st);
    if (rc) return rc;
    return transpose_inner(dxt, dx, 1, in_f, batch, st);                        // (in, batch) -> (batch, in)
}

int tc_fc_wgrad_small_batch(int batch, int in_f, int out_f, const void* x, const void* dy, void* dw, void* db, void* ws, size_t ws_bytes,
                            cudaStream_t st)
{
    float* xt; void* inner; size_t inner_bytes;
    if (!fc_ws(batch, in_f, ws, ws_bytes, &xt, &inner, &inner_bytes)) return B2C_ERR_WORKSPACE_TOO_SMALL;
    if (((uintptr_t)x | (uintptr_t)dy | (uintptr_t)dw) & 15) return B2C_ERR_MISALIGNED;
    int rc = transpose_inner(x, xt, 1, batch, in_f, st);
    if (rc) return rc;
    rc = tc_fprop_nhwc(fc_pixels_view(in_f, batch, out_f, B2C_W_CRSK), xt, dy, nullptr, nullptr, 0, dw, inner, inner_bytes, st);
    if (rc || !db) return rc;
    return channel_sum(B2C_F32, B2C_LAYOUT_NHWC, batch, out_f, 1, dy, db, inner, inner_bytes, st);
}

#ifdef B2C_TC_PROFILE
extern "C" int b2c_debug_prof(long long* out, int reset)
{
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out, g_tc_prof, sizeof(long long) * 32);
    if (reset) { long long z[32] = {0}; cudaMemcpyToSymbol(g_tc_prof, z, sizeof(z)); }
    return 0;
}
#endif

// Self-test of the bounded wait: one warp waits on a barrier nothing arrives at, with a short limit; the wait gives
// up, records TC_ERR_SELFTEST in the status word and the kernel returns.  Exercises the path the convolution
// kernels take when a wait runs out, without anything being wrong.
__global__ void tc_wait_selftest_kernel(long long limit_cycles)
{
    pdl_prologue();
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) { mbar_init(&bar, 1); abort_flag = 0; fence_barrier_init(); }
    __syncthreads();
    mbar_wait(&bar, 0, &abort_flag, &g_tc_status, TC_ERR_SELFTEST, limit_cycles);
}

int tc_wait_selftest(long long limit_cycles, cudaStream_t st)
{
    if (limit_cycles < 1 || limit_cycles > TC_WAIT_CYCLES) return B2C_ERR_BAD_GEOMETRY;
    launch_pdl(tc_wait_selftest_kernel, 1, 32, 0, st, limit_cycles);
    return check_launch("tc_wait_selftest_kernel");
}

int tc_read_status(int* out)
{
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int));
    if (e != cudaSuccess) { set_cuda_error(e, "cudaMemcpyFromSymbol(g_tc_status)"); return B2C_ERR_CUDA; }
    if (v != 0) {
        // a kernel that gave up may have left hand-over flags behind: return every bank to zeros
        int zero = 0;
        cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int));
        void* sync = nullptr;
        if (cudaGetSymbolAddress(&sync, g_tc_sync) == cudaSuccess && sync) cudaMemset(sync, 0, sizeof(unsigned int) * TC_SYNC_BANKS * TC_SYNC_WORDS);
    }
    *out = v;
    return B2C_OK;
}

}  // namespace b2c

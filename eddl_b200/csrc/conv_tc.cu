// Conv2D forward / backward-data / backward-weight as ONE implicit-GEMM kernel on the
// Blackwell tensor cores: tcgen05.mma (kind::tf32, cta_group::1, M=128) with the fp32
// accumulator in tensor memory, operands staged in shared memory in the canonical K-major
// SWIZZLE_128B layout, mbarrier producer/consumer pipeline, tcgen05.ld epilogue.
// Replaces gpu_im2col_k + cublasSgemm + gpu_traspose_batch_depth of EDDL
// (src/hardware/gpu/nn/gpu_conv.cu:159-372); the contraction is cpu_conv2D / cpu_conv2D_grad /
// cpu_conv2D_back (src/hardware/cpu/nn/cpu_conv.cpp:114-280).
//
// GEMM view (D[m][n] = sum_k A[m][k] * B[n][k], 128 x BN output tile per CTA):
//   forward          m = output pixel (n,p,q)   n = filter        k = (c,r,s)   A = x gathered, B = w
//   backward-data    m = input pixel (n,y,x)    n = in-channel    k = (f,r,s)   A = dy gathered, B = w
//   backward-weight  m = (c,r,s)                n = filter        k = (n,p,q)   A = x gathered, B = dy
// In all three the address of an operand element separates into a row part plus a k part
// (src[rowOff[row] + kOff[k]]) and zero padding is the test 0 <= rowY+kY < limY, 0 <= rowX+kX < limX,
// so small index tables built by a set-up kernel drive a single gather routine: no im2col
// buffer, no col2im atomics, no layout transposes.  Pixels sit on the M (TMEM lane) axis, so the
// epilogue's stores are coalesced along the NCHW pixel dimension.
//
// fp32-equivalent mode (precision 0) is the 3xTF32 split: every operand value v is staged as
// hi = v with the 13 low mantissa bits cleared and lo = v - hi (exact), and each k-step issues
// hi*hi + lo*hi + hi*lo into the same fp32 accumulator.  precision 1 issues hi*hi only.  precision 2 keeps the
// TF32 hi*hi chain and computes the two cross terms as ONE bf16 MMA chain ([lo | hi] x [hi | lo] concatenated along k,
// a third fewer tensor-core and shared-memory cycles); its error is about four times that of precision 0 (bf16 rounding
// of the cross-term operands, ~2^-20 per product), still inside 1e-5, and it is opt-in.
//
// The tensor core adds each MMA into the fp32 accumulator with truncation, so a long chain of
// accumulations drifts toward zero in proportion to its length (measured: 3e-5 relative at K = 4096
// with a single accumulator).  The kernel therefore keeps FOUR accumulators of BN columns in tensor
// memory: the dominant hi*hi products rotate over three of them k-step by k-step (chain length K/24)
// and the two small cross terms go to the fourth; the epilogue adds the four in fp32 with rounding.
//
// Operand feeding.  The weight operand of forward / backward-data is pre-split and pre-swizzled once per
// call (pack_b_kernel) and every stage fetches its tile with ONE TMA bulk copy (cp.async.bulk, completion on
// the stage's mbarrier).  The activation operand is gathered by the producer warps with ordinary coalesced
// loads rather than TMA tensor copies: the tap offset (s - pad) of an NCHW row is not a multiple of 16
// bytes, which a tiled TMA copy requires, and the hi/lo split needs a pass through registers anyway.
// Backward-weight gathers both operands: whatever is contiguous along k = (n, p, q) inside an image (dy always, x for 1x1
// stride-1 layers) is read with 16-byte loads, a quarter warp per 128-byte row, so every load and store instruction touches
// four whole rows; the tap-shifted x operand of larger filters keeps one lane per k.
// Every wait on an mbarrier is bounded; on time-out the kernel records a status code, leaves
// its loops, frees its tensor memory and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <array>
#include <map>
#include <mutex>
#include <type_traits>
#include <vector>
#include "common.cuh"
#include "conv_common.cuh"

namespace {

using namespace eb;

constexpr int BM = 128;             // UMMA M (TMEM lanes)
constexpr int BK = 32;              // fp32 per 128-byte swizzle row
constexpr int NPROD = 256;          // producer threads (warps 0-7); warp 8 issues the MMAs; warps 9-12 run the epilogue
constexpr int NEPI = 128;           // epilogue threads (warps 9-12)
constexpr int NTHREADS = NPROD + 32 + NEPI + 32;     // + warp 13: L2 prefetch of the activation operand / TMA issue
// TMA-fed forward / backward-data kernels run a second set of four epilogue warps (warps 14-17): their short-reduction,
// output-heavy layers are bound by the epilogue's chain of tensor-memory reads, and two warps per lane quarter halve it
constexpr int NTHREADS_ATMA = NTHREADS + NEPI;
constexpr int threads_of(int tma) { return (tma == 1 || tma == 3) ? NTHREADS_ATMA : NTHREADS; }
// backward-weight of 3x3 stride-1 pad-1 layers fed from raw slabs (TMA = 4): a tile's 128 rows are the nine taps of 14 channels
// (126 rows, the last two stay zero) and a K-block is 32 pixels of one image; one slab of [16 channels][152 pixels] -- the 32
// pixels plus a halo of W + 1 either side, its start rounded down to 16 bytes -- serves all 126 rows (W <= 57)
constexpr int WS_CH = 14, WS_ROWS = 9 * WS_CH, WS_SLAB_PX = 152, WS_SLAB_CH = 16;
constexpr int SLAB_PX = 256;        // pixels per channel of a raw slab (3x3 TMA-fed kernels): 128 rows + a halo of W + 1 either side + alignment
constexpr int PF_AHEAD = 8;         // K-blocks the prefetch warp may run ahead of the producers
constexpr int INVALID_Y = -20000;
constexpr int NMAIN = 3;             // rotating hi*hi accumulators; a fourth holds the cross terms

struct TcParams {
    const float *srcA, *srcB;
    float *out;
    const float *bias;      // per n (forward only), may be null
    const int2 *rowA;       // [M_total]  .x = offset part, .y = (y << 16) | (x & 0xffff)
    const int2 *kA;         // [K_pad]
    const int *kC;          // [K_pad]  compact form of kA for check 0 (offset) and check 1 ((offset << 5) | tap)
    const int *rowB;        // [N_total]
    const int *kB;          // [K_pad]    -1 = beyond K_total
    const int *outM;        // [M_total]
    int out_n_stride;
    int M_total, N_total, K_pad;
    int tiles_m, tiles_n, splits;
    int limY, limX;
    int kblocks_per_split;
    long long split_stride; // elements between the partial outputs of consecutive splits
    int accumulate;
    int add_zero;           // plain stores write 0 + v (the bits a read-modify-write into zeros would leave)
    int check;              // padding test of the gathered operand: 0 none needed, 1 per-row tap bitmask, 2 coordinates
    const float *packedB;   // forward / backward-data: pre-split, pre-swizzled B tiles [kblock][n tile][hi|lo][BN x 32]
    int nmain;              // rotating hi*hi accumulators in use: 1 for short chains, NMAIN otherwise
    int pf_rows;            // > 0: warp 13 prefetches the A operand into L2, one line per pf_rows tile rows and k (0 = off)
    int *status;
    // TMA-fed 1x1 stride-1 layers (ATMA kernels): the activation tensor and the output tensor as [image][channel][pixel]
    // tensor maps with boxes of 32 pixels x 32 channels; a tile row is a pixel of a 32-pixel CHUNK of one image, so the row
    // space is images x chunks_per_image x 32 (rows past the end of an image are zero on the way in and clipped on the way out)
    int chunks_per_image, images;
    int reduce_out;         // the output is added into (TMA reduce) instead of stored
    int img_w;              // STMA: width of the image plane (the halo of a slab is img_w + 1 pixels either side)
    int tap_sign;           // STMA: +1 forward (tap (r, s) reads pixel + (r-1, s-1)), -1 backward-data (pixel + (1-r, 1-s))
    int raw_hi;             // WTMA: leave the landed fp32 values as the hi plane (the tensor core reads only their upper 19 bits)
    int plane_px;           // WSLAB: pixels of an image plane
    alignas(64) CUtensorMap mapA;
    alignas(64) CUtensorMap mapOut;
};

// ---- PTX wrappers ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up after ~2 s of SM clock, or as soon as another role of the CTA has given up (the abort flag), and
// reports false.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; i++) if (mbar_try(bar, parity)) return true;
        if (*abort_flag || clock64() - t0 > 4000000000LL) return false;
    }
}
// The same for a whole warp: every lane waits, and the warp leaves together if any lane gave up, so that no warp-wide
// (.sync.aligned, shuffle) instruction that follows is reached by part of a warp.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag)) != 0;
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// TMA bulk copy global -> shared (1-D, 16-byte aligned, size a multiple of 16), completion counted on an mbarrier
__device__ __forceinline__ void tma_bulk_g2s(uint32_t dst_smem, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// TMA tensor copy global -> shared: a [1][32 channels][32 pixels] box of a 3-D tensor map; coordinates may lie outside the
// tensor (the missing elements arrive as zeros), x must be a multiple of 4 elements
__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const CUtensorMap *map, int x, int y, int z, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst_smem), "l"((uint64_t)map), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}
// TMA tensor copy shared -> global (elements outside the tensor are dropped), plain store or fp32 add into global memory
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, int x, int y, int z, uint32_t src_smem) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];"
                 ::"l"((uint64_t)map), "r"(x), "r"(y), "r"(z), "r"(src_smem) : "memory");
}
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap *map, int x, int y, int z, uint32_t src_smem) {
    asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2, %3}], [%4];"
                 ::"l"((uint64_t)map), "r"(x), "r"(y), "r"(z), "r"(src_smem) : "memory");
}
__device__ __forceinline__ void tma_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void tma_wait_group_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
template <int N> __device__ __forceinline__ void tma_wait_group() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// K-major SWIZZLE_128B shared-memory matrix descriptor: rows of 128 bytes, 8-row groups 1024 bytes
// apart (stride byte offset), descriptor version 1, layout type 2, 1024-byte aligned tile base.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// fp32 accumulate, TF32 x TF32, both operands K-major, M = 128, N = bn
__host__ __device__ constexpr uint32_t make_idesc(int bn) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

// fp32 accumulate, BF16 x BF16 (kind::f16), both operands K-major, M = 128, N = bn, K = 16 per instruction
__host__ __device__ constexpr uint32_t make_idesc_bf16(int bn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

// byte offset of 16-byte chunk `chunk` of row `row` inside a [rows][128 bytes] SWIZZLE_128B tile
__device__ __forceinline__ uint32_t swz_chunk(uint32_t row, uint32_t chunk) { return row * 128u + (((chunk ^ row) & 7u) << 4); }
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);          // a in the low half = the lower address
    return *reinterpret_cast<const uint32_t *>(&v);
}

__device__ __forceinline__ void split_tf32(float v, float &hi, float &lo) {
    hi = __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
    lo = __fsub_rn(v, hi);
}

// byte offset of element (row, k) inside a [rows][32 fp32] SWIZZLE_128B tile
__device__ __forceinline__ uint32_t swz(uint32_t row, uint32_t k) {
    return row * 128u + ((((k >> 2) ^ row) & 7u) << 4) + ((k & 3u) << 2);
}

// Shared memory of a CTA.  Gather kernels: the operand ring only.  ATMA kernels add a ring of RAW_STAGES raw activation
// tiles ([4 chunks][32 channels][32 pixels] fp32, written by TMA) in front of the converters and two 4 KB staging buffers
// per epilogue warp behind them, and keep a shorter operand ring in exchange.
template <int BN_, bool SPLIT3, bool ATMA = false, bool WSLAB = false>
struct Layout {
    static constexpr int A_BYTES = BM * BK * 4;
    static constexpr int B_BYTES = BN_ * BK * 4;
    static constexpr int STAGE_BYTES = (A_BYTES + B_BYTES) * (SPLIT3 ? 2 : 1);
    static constexpr int RAW_BYTES = BM * BK * 4;                  // one K-block of raw activations
    static constexpr int RAW_STAGES = ATMA ? 4 : 0;
    static constexpr int OUT_BYTES = ATMA ? 8 * 32 * 32 * 4 : 0;       // one 32 x 32 staging block per epilogue warp
    // 227 KB per CTA minus the alignment slack and the barrier words; gather kernels keep their 200 KB ring
    static constexpr int WSLAB_BYTES = WSLAB ? WS_SLAB_CH * WS_SLAB_PX * 4 : 0;    // one raw slab of x beside every stage
    static constexpr int RING_BUDGET = ATMA ? 232448 - 1024 - 256 - RAW_STAGES * RAW_BYTES - OUT_BYTES : (WSLAB ? 232448 - 1024 - 256 : 200 * 1024);
    static constexpr int STAGES = (RING_BUDGET / (STAGE_BYTES + WSLAB_BYTES)) > 4 ? 4 : (RING_BUDGET / (STAGE_BYTES + WSLAB_BYTES));
    static_assert(STAGES >= 2, "the operand ring needs two stages");
    static constexpr int TABLE_BYTES = (ATMA || WSLAB) ? 0 : 8 * 32 * 12;     // backward-weight: 32 row entries of A (8 bytes) and of B (4 bytes) per producer warp
    static constexpr int SMEM_BYTES = 1024 /*alignment slack*/ + STAGES * (STAGE_BYTES + WSLAB_BYTES) + RAW_STAGES * RAW_BYTES + OUT_BYTES + TABLE_BYTES + 256;
    static_assert(SMEM_BYTES <= 232448, "shared memory of a CTA");
};

// Shared memory of the TMA-fed backward-weight kernels (WTMA, WSLAB).  What TMA delivers -- the dy tile in its final place
// as the hi plane of B, and the x tile as the hi plane of A (WTMA) or the raw slab of x (WSLAB) -- lives in a HI ring that is
// as deep as shared memory allows: a copy takes about 2700 cycles from issue to landing (measured, L2 hits included), twice
// the 1284 cycles of a K-block's MMAs, so three or more K-blocks must be in flight beside the one being converted and the one
// being multiplied.  What the producer warps compute -- the lo planes, and for WSLAB the whole A operand -- lives in a LO ring
// of two slots, one per producer group: it is occupied only from the conversion to the end of the K-block's MMAs.
template <int BN_, bool SPLIT3, bool WSLAB>
struct WLayout {
    static constexpr int A_BYTES = BM * BK * 4;
    static constexpr int B_BYTES = BN_ * BK * 4;
    static constexpr int X_BYTES = WSLAB ? WS_SLAB_CH * WS_SLAB_PX * 4 : A_BYTES;       // what lands beside the dy tile
    static constexpr int LO_BYTES = WSLAB ? (SPLIT3 ? 2 : 1) * A_BYTES + (SPLIT3 ? B_BYTES : 0) : (SPLIT3 ? A_BYTES + B_BYTES : 0);
    static constexpr int LO_SLOTS = 2;
    static constexpr int BUDGET = 232448 - 1024 - 256 - LO_SLOTS * LO_BYTES;
    static constexpr int HI_SLOTS = BUDGET / (B_BYTES + X_BYTES) > 6 ? 6 : BUDGET / (B_BYTES + X_BYTES);
    static_assert(HI_SLOTS >= 3, "the landing ring needs three slots");
    static constexpr int SMEM_BYTES = 1024 + HI_SLOTS * (B_BYTES + X_BYTES) + LO_SLOTS * LO_BYTES + 256;
};

// Persistent, warp-specialised kernel: each CTA walks tiles t = blockIdx.x, blockIdx.x + gridDim.x, ... of the
// (split, filter tile, row tile) space.
//   warps 0-7   producers: gather / split / store the A tile (and B for backward-weight).  Forward / backward-data: two
//               groups of four warps take alternate K-blocks, and the first thread of a group issues the TMA bulk copy
//               of that block's packed weight tile.  The shared-memory ring keeps running across tile boundaries.
//   warp  8     one lane issues the MMAs of a tile into one of the accumulator SETS in tensor memory.
//   warps 9-12  epilogue: drain a finished set (tcgen05.ld), add its accumulators, store -- overlapped with the MMAs of
//               the next tile whenever tensor memory holds two sets (BN <= 64, or short chains at BN = 128).
//   warp  13    1x1 unpadded forward / backward-data only: prefetches the activation operand of coming K-blocks into L2.
// WGRAD = false (forward, backward-data): A rows are pixels (one thread per row, vector stores); B is the weight operand,
// prepared once per call by pack_b_kernel.  WGRAD = true (backward-weight): A and B are gathered with one lane per k.
// BGATHER (backward-weight of 1x1 stride-1 unpadded convolutions): both operands are contiguous along k = (n, p, q) inside an
// image, so the producers gather BOTH with 16-byte loads -- eight lanes per 128-byte row, four rows per instruction -- and no TMA.
// ATMA (forward / backward-data of 1x1 stride-1 unpadded convolutions whose planes are a multiple of 4 pixels): the
// activation operand is not gathered from global memory.  Warp 13 issues TMA tensor copies of raw [32 channels x 32 pixels]
// boxes into a ring that runs several K-blocks ahead (the gather's one-K-block-per-round-trip latency bound is gone), the
// producer warps read their rows out of that ring instead of global memory, and the epilogue warps hand 32 x 32 output
// blocks to TMA stores (or TMA fp32 adds) through shared memory instead of issuing one 128-byte store per column.
// WTMA (TMA = 2: backward-weight of the same layers): both operands are [image][channel][pixel] tensors whose rows are
// contiguous along k = (image, pixel), so warp 13 lets TMA write them straight into the operand ring in the K-major
// SWIZZLE_128B layout the MMA reads (a K-block = 32 pixels of one image; pixels past the end of the image arrive as
// zeros and add nothing), and the producer warps only split what has landed into its hi / lo planes, in place.
template <int BN_, int PREC, bool WGRAD, bool BGATHER = false, int TMA = 0>
__global__ void __launch_bounds__(threads_of(TMA), 1) igemm_tc_kernel(const __grid_constant__ TcParams P) {
    constexpr bool STMA = TMA == 3;                      // 3x3 stride-1 pad-1 layers fed from raw slabs (see load_row)
    constexpr bool ATMA = TMA == 1 || STMA, WTMA = TMA == 2, WSLAB = TMA == 4;
    static_assert(!(WTMA || WSLAB) || (!WGRAD && BGATHER), "the TMA-fed backward-weight variants replace the both-operands gather");
    constexpr bool SPLIT3 = PREC != 1;                   // operands staged as hi / lo planes
    constexpr bool CROSS_BF16 = PREC == 2 && !WGRAD && !BGATHER;     // cross terms as one bf16 MMA chain
    static_assert(!ATMA || (!WGRAD && !BGATHER), "the TMA-fed variant covers forward and backward-data");
    using L = Layout<BN_, SPLIT3, ATMA, WSLAB>;
    constexpr int STAGES = L::STAGES;
    constexpr int RAWS = L::RAW_STAGES;
    constexpr bool A_ROWMAJOR = !WGRAD;
    constexpr bool B_TMA = !WGRAD && !BGATHER;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *stage_base = smem;
    uint8_t *raw_base = smem + STAGES * L::STAGE_BYTES;                       // ATMA: raw activation ring; WSLAB: one slab per stage
    static_assert(!WSLAB || RAWS == 0, "the slab ring of backward-weight takes the place of the raw ring");
    uint8_t *out_base = raw_base + RAWS * L::RAW_BYTES + STAGES * L::WSLAB_BYTES;      // ATMA: epilogue staging, 2 x 4 KB per warp
    // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], then ATMA: raw_full[RAWS], raw_empty[RAWS]; WTMA: landed[STAGES]
    uint8_t *table_base = out_base + L::OUT_BYTES;                            // backward-weight: per-warp row tables
    constexpr bool WMODE = WTMA || WSLAB;
    static_assert(!WMODE || (2 * STAGES + 4 + 2 * WLayout<BN_, SPLIT3, WSLAB>::HI_SLOTS) * 8 + 16 <= 256, "barrier words");
    using WL = WLayout<BN_, SPLIT3, WSLAB>;
    constexpr int HS = WMODE ? WL::HI_SLOTS : 0;
    // WMODE: [dy tiles: HS x B_BYTES][LO ring: 2 x LO_BYTES][x tiles or slabs: HS x X_BYTES], all swizzled tiles 1024-byte aligned
    uint8_t *w_hib = smem, *w_lo = smem + HS * WL::B_BYTES, *w_x = w_lo + WL::LO_SLOTS * WL::LO_BYTES;
    if constexpr (WMODE) table_base = w_x + HS * WL::X_BYTES;       // the barrier words follow
    constexpr int XBARS = WMODE ? 2 * HS : 2 * RAWS;
    uint64_t *bars = (uint64_t *)(table_base + (WMODE ? 0 : L::TABLE_BYTES));
    uint32_t *tmem_slot = (uint32_t *)(bars + 2 * STAGES + 4 + XBARS);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);
    volatile int *progress = abort_flag + 1;              // last K-block (CTA sequence number) producer group 0 has stored

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kb_total = P.K_pad / BK;
    const int tiles_mn = P.tiles_m * P.tiles_n;
    const int total_tiles = tiles_mn * P.splits;
    // accumulators per set: the rotating hi*hi ones plus (3xTF32) the cross-term one
    const int nacc = P.nmain + (SPLIT3 ? 1 : 0);
    const int nsets = (512 / (nacc * BN_)) >= 2 ? 2 : 1;
    const int small_off = P.nmain * BN_;                 // column offset of the cross-term accumulator inside a set
    const int set_cols = nacc * BN_;

    const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + STAGES);
    const uint32_t bar_acc_full = smem_u32(bars + 2 * STAGES), bar_acc_empty = smem_u32(bars + 2 * STAGES + 2);
    const uint32_t bar_raw_full = smem_u32(bars + 2 * STAGES + 4), bar_raw_empty = smem_u32(bars + 2 * STAGES + 4 + RAWS);

    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(bar_full + 8 * s, NPROD / 64 + (B_TMA ? 1 : 0)); mbar_init(bar_empty + 8 * s, 1); }
        for (int s = 0; s < 2; s++) { mbar_init(bar_acc_full + 8 * s, 1); mbar_init(bar_acc_empty + 8 * s, (ATMA ? 2 : 1) * NEPI / 32); }
        // a raw tile is filled by one expect_tx arrival plus the TMA bytes, and released by the four warps of the group that read it
        // (a slab serves nine K-blocks shared by both groups: all eight producer warps release it)
        for (int s = 0; s < RAWS; s++) { mbar_init(bar_raw_full + 8 * s, 1); mbar_init(bar_raw_empty + 8 * s, STMA ? 8 : 4); }
        // WMODE: landed[HS] (one expect_tx arrival + the bytes) and hi_empty[HS] (one commit of the MMA thread)
        if constexpr (WMODE) for (int s = 0; s < 2 * HS; s++) mbar_init(bar_raw_full + 8 * s, 1);
        *abort_flag = 0;
        *progress = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool failed = false;
    int fail_code = 0;          // which wait gave up (numbered in source order), reported through the status word

    // K-block range of a tile's split
    auto kb_range = [&](int t, int &kb0, int &nkb) {
        const int split = t / tiles_mn;
        kb0 = split * P.kblocks_per_split;
        nkb = min(kb_total, kb0 + P.kblocks_per_split) - kb0;
    };

    if (warp < 8) {
        // ============================ producers ============================
        constexpr uint32_t B_IMAGE = (uint32_t)L::B_BYTES * (SPLIT3 ? 2u : 1u);
        if constexpr (WTMA) {
            // The raw fp32 tiles of K-block g have landed in HI slot g % HS, already swizzled by the copy: they ARE the hi planes
            // (the tensor core reads only the upper 19 bits of a TF32 operand).  The group's 128 threads walk them 16 bytes at a
            // time -- the split is elementwise, so the swizzle does not matter -- and write lo = v - hi into the group's LO slot
            // (and, unless raw_hi, hi back in place).
            const int group = warp >> 2, gtid = tid & 127;
            int t = blockIdx.x, kb0 = 0, nkb = 0, it = group;
            auto settle = [&]() {
                while (t < total_tiles) {
                    kb_range(t, kb0, nkb);
                    if (it < nkb) return;
                    it -= nkb; t += gridDim.x;
                }
            };
            settle();
            for (int g = group; t < total_tiles; g += 2) {
                const int h = g % HS, l = group;
                if (!mbar_wait_warp(bar_raw_full + 8 * h, (g / HS) & 1, abort_flag)) { failed = true, fail_code = 1; break; }
                if (!mbar_wait_warp(bar_empty + 8 * l, ((g >> 1) & 1) ^ 1, abort_flag)) { failed = true, fail_code = 2; break; }
                if constexpr (SPLIT3) {
                    uint8_t *lo_slot = w_lo + l * WL::LO_BYTES;
                    // all of a plane's loads go out before its first store: the compiler cannot move a shared-memory load above
                    // an earlier shared-memory store, so load / split / store per piece would cost one load latency per piece
                    auto split_plane = [&](uint8_t *hi_plane, uint8_t *lo_plane, auto bytes_c) {
                        constexpr int PIECES = decltype(bytes_c)::value / (128 * 16);
                        float4 v[PIECES];
#pragma unroll
                        for (int i = 0; i < PIECES; i++) v[i] = *(const float4 *)(hi_plane + (gtid + 128 * i) * 16);
#pragma unroll
                        for (int i = 0; i < PIECES; i++) {
                            float4 hi, lo;
                            split_tf32(v[i].x, hi.x, lo.x); split_tf32(v[i].y, hi.y, lo.y); split_tf32(v[i].z, hi.z, lo.z); split_tf32(v[i].w, hi.w, lo.w);
                            *(float4 *)(lo_plane + (gtid + 128 * i) * 16) = lo;
                            if (!P.raw_hi) *(float4 *)(hi_plane + (gtid + 128 * i) * 16) = hi;
                        }
                    };
                    split_plane(w_x + h * WL::X_BYTES, lo_slot, std::integral_constant<int, WL::A_BYTES>{});
                    split_plane(w_hib + h * WL::B_BYTES, lo_slot + WL::A_BYTES, std::integral_constant<int, WL::B_BYTES>{});
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_full + 8 * l);
                it += 2; settle();
            }
        } else if constexpr (WSLAB) {
            // K-block g of the CTA's sequence has landed in HI slot g % HS: the dy tile (the hi plane of B, already swizzled by the
            // copy) and the raw slab of x.  Warp wq of the group builds rows [32 wq, 32 wq + 32)
            // of A -- row r = tap r % 9 of channel r / 9 -- with one lane per pixel: the value is the slab element at the
            // pixel's position shifted by the tap, or zero where the tap leaves the image row (left / right edge; above and
            // below the image the copy delivered zeros) or the pixel lies past the end of the plane.  Then the group splits B.
            const int group = warp >> 2, wq = warp & 3, gtid = tid & 127;
            const int W = P.img_w, cpi = P.chunks_per_image;
            int tab[32];                        // (slab offset of the row's tap relative to the pixel) << 2 | which edge masks it
#pragma unroll
            for (int j = 0; j < 32; j++) {
                const int r = wq * 32 + j, c_rel = r / 9, tap = r - 9 * c_rel, tr = tap / 3, ts = tap - 3 * tr;
                tab[j] = r < WS_ROWS ? (c_rel * WS_SLAB_PX + (tr - 1) * W + (ts - 1)) * 4 + ts : 3;      // kind 3: a row that stays zero
            }
            uint32_t so[8];                     // this lane's byte offset inside a swizzled row whose number is e modulo 8
#pragma unroll
            for (int e = 0; e < 8; e++) so[e] = (uint32_t)(((((lane >> 2) ^ e) & 7) << 4) + ((lane & 3) << 2));
            int t = blockIdx.x, kb0 = 0, nkb = 0, it = group;
            auto settle = [&]() {
                while (t < total_tiles) {
                    kb_range(t, kb0, nkb);
                    if (it < nkb) return;
                    it -= nkb; t += gridDim.x;
                }
            };
            settle();
            for (int g = group; t < total_tiles; g += 2) {
                const int h = g % HS, l = group;
                if (!mbar_wait_warp(bar_raw_full + 8 * h, (g / HS) & 1, abort_flag)) { failed = true, fail_code = 3; break; }
                if (!mbar_wait_warp(bar_empty + 8 * l, ((g >> 1) & 1) ^ 1, abort_flag)) { failed = true, fail_code = 4; break; }
                const int x0 = ((kb0 + it) % cpi) * 32;
                const int base = ((x0 - W - 1 + 4096) & ~3) - 4096;
                const int px = x0 + lane, q = px % W;
                const bool inside = px < P.plane_px;
                // bit `kind` set = rows of that kind are zero for this lane: 0 left neighbour, 1 same column, 2 right neighbour, 3 always
                const unsigned zero_bits = ((!inside || q == 0) ? 1u : 0u) | (!inside ? 2u : 0u) | ((!inside || q == W - 1) ? 4u : 0u) | 8u;
                const float *slab = (const float *)(w_x + h * WL::X_BYTES) + (x0 - base + lane);
                uint8_t *sA_hi = w_lo + l * WL::LO_BYTES + wq * (32 * 128);
                uint8_t *sA_lo = sA_hi + WL::A_BYTES;                     // only when SPLIT3
                // all loads before the first store (a shared-memory load cannot be moved above an earlier shared-memory store)
                float av[32];
#pragma unroll
                for (int j = 0; j < 32; j++) av[j] = slab[tab[j] >> 2];
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    const float v = ((zero_bits >> (tab[j] & 3)) & 1u) ? 0.f : av[j];
                    const uint32_t off = (uint32_t)(j * 128) + so[j & 7];
                    if (SPLIT3) { float hi, lo; split_tf32(v, hi, lo); *(float *)(sA_hi + off) = hi; *(float *)(sA_lo + off) = lo; }
                    else *(float *)(sA_hi + off) = v;
                }
                if constexpr (SPLIT3) {
                    uint8_t *sB_hi = w_hib + h * WL::B_BYTES, *sB_lo = w_lo + l * WL::LO_BYTES + 2 * WL::A_BYTES;
                    constexpr int PIECES = WL::B_BYTES / (128 * 16);
                    float4 bv[PIECES];
#pragma unroll
                    for (int i = 0; i < PIECES; i++) bv[i] = *(const float4 *)(sB_hi + (gtid + 128 * i) * 16);
#pragma unroll
                    for (int i = 0; i < PIECES; i++) {
                        float4 hi, lo;
                        split_tf32(bv[i].x, hi.x, lo.x); split_tf32(bv[i].y, hi.y, lo.y); split_tf32(bv[i].z, hi.z, lo.z); split_tf32(bv[i].w, hi.w, lo.w);
                        *(float4 *)(sB_lo + (gtid + 128 * i) * 16) = lo;
                        if (!P.raw_hi) *(float4 *)(sB_hi + (gtid + 128 * i) * 16) = hi;
                    }
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_full + 8 * l);
                it += 2; settle();
            }
        } else if constexpr (BGATHER && !WGRAD) {
            // Two groups of four warps on alternate K-blocks, as below.  Warp wq of a group gathers rows [32 wq, 32 wq + 32) of
            // A and its share of B: a quarter warp covers one 128-byte row (lane & 7 = the 16-byte chunk), so every load
            // instruction reads four whole rows, coalesced, and every store instruction fills four whole swizzle rows.
            const int group = warp >> 2, wq = warp & 3, sub = lane >> 3, chunk = lane & 7;
            constexpr int BROWS = BN_ / 4, BI = BROWS / 4;        // B rows per warp and load instructions for them
            int offA[8], offB[BI], rows_of = -1;
            float4 a4[8], b4[BI];
            auto load = [&](int mn, int kblock) {
                if (mn != rows_of) {
                    rows_of = mn;
                    const int m0 = (mn % P.tiles_m) * BM, n0 = (mn / P.tiles_m) * BN_;
#pragma unroll
                    for (int i = 0; i < 8; i++) { const int m = m0 + wq * 32 + 4 * i + sub; offA[i] = m < P.M_total ? __ldg(P.rowA + m).x : 0; }
#pragma unroll
                    for (int i = 0; i < BI; i++) { const int n = n0 + wq * BROWS + 4 * i + sub; offB[i] = n < P.N_total ? __ldg(P.rowB + n) : 0; }
                }
                // groups of four k are contiguous and 16-byte aligned in both tensors (checked by the dispatcher)
                const float *pa = P.srcA + __ldg(P.kC + kblock * BK + chunk * 4);
                const float *pb = P.srcB + __ldg(P.kB + kblock * BK + chunk * 4);
#pragma unroll
                for (int i = 0; i < 8; i++) a4[i] = ldg4(pa + offA[i]);
#pragma unroll
                for (int i = 0; i < BI; i++) b4[i] = ldg4(pb + offB[i]);
            };
            auto put = [&](uint8_t *hi_plane, uint8_t *lo_plane, int row, float4 v) {
                const uint32_t off = swz(row, chunk * 4);
                if (SPLIT3) {
                    float4 hi, lo;
                    split_tf32(v.x, hi.x, lo.x); split_tf32(v.y, hi.y, lo.y); split_tf32(v.z, hi.z, lo.z); split_tf32(v.w, hi.w, lo.w);
                    *(float4 *)(hi_plane + off) = hi; *(float4 *)(lo_plane + off) = lo;
                } else {
                    *(float4 *)(hi_plane + off) = v;
                }
            };
            auto store = [&](int s) {
                uint8_t *sA_hi = stage_base + s * L::STAGE_BYTES;
                uint8_t *sA_lo = sA_hi + L::A_BYTES;                      // only when SPLIT3
                uint8_t *sB_hi = sA_hi + (SPLIT3 ? 2 : 1) * L::A_BYTES;
                uint8_t *sB_lo = sB_hi + L::B_BYTES;
#pragma unroll
                for (int i = 0; i < 8; i++) put(sA_hi, sA_lo, wq * 32 + 4 * i + sub, a4[i]);
#pragma unroll
                for (int i = 0; i < BI; i++) put(sB_hi, sB_lo, wq * BROWS + 4 * i + sub, b4[i]);
            };
            int t = blockIdx.x, kb0 = 0, nkb = 0, it = group;
            auto settle = [&]() {
                while (t < total_tiles) {
                    kb_range(t, kb0, nkb);
                    if (it < nkb) return;
                    it -= nkb; t += gridDim.x;
                }
            };
            settle();
            if (t < total_tiles) load(t % tiles_mn, kb0 + it);
            for (int g = group; t < total_tiles; g += 2) {
                const int s = g % STAGES;
                const uint32_t par = ((g / STAGES) & 1) ^ 1;
                if (!mbar_wait_warp(bar_empty + 8 * s, par, abort_flag)) { failed = true, fail_code = 5; break; }
                store(s);
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_full + 8 * s);
                it += 2; settle();
                if (t < total_tiles) load(t % tiles_mn, kb0 + it);
            }
        } else if constexpr (A_ROWMAJOR) {
            // Two groups of four warps work on alternate K-blocks (group 0 the even ones of the CTA's K-block
            // sequence, group 1 the odd ones), one thread per tile row and all 32 k of the block per thread.
            // The groups drift out of phase, so one group's loads are in flight while the other splits and stores.
            const int group = warp >> 2;
            const int arow = tid & (BM - 1);
            float av[BK];
            int2 myRow = make_int2(0, INVALID_Y << 16);
            int ry = INVALID_Y, rx = 0, row_tile = -1;

            // STMA state of this thread's row: position of the row inside the slab for the centre tap, and whether the row's
            // pixel sits on the left / right edge of the image (its horizontal neighbours then lie in another image row)
            int slab_pos = 0; bool edge_l = false, edge_r = false;
            auto load_row = [&](int t, int kb0, int it, int gseq) -> bool {
                if constexpr (STMA) {
                    // K-blocks come as (32-channel group, tap): the nine taps of a group read the SAME raw slab
                    // [32 channels][SLAB_PX pixels] -- the tile's 128 pixels plus a halo of img_w + 1 pixels either side --
                    // each at its own shift, so the activations cross from L2 to shared memory once instead of nine times.
                    // Pixels before the first / after the last image row are outside the tensor and arrive as zeros; a
                    // horizontal neighbour outside the row is masked here.
                    const int mn = t % tiles_mn;
                    if (mn != row_tile) {
                        row_tile = mn;
                        const int tile_in_image = (mn % P.tiles_m) % (P.chunks_per_image / 4);
                        const int t0 = tile_in_image * BM;
                        const int base = ((t0 - P.img_w - 1 + 4096) & ~3) - 4096;         // rounded down to 16 bytes, may be negative
                        slab_pos = t0 - base + arow;
                        const int q = (t0 + arow) % P.img_w;
                        edge_l = q == 0; edge_r = q == P.img_w - 1;
                    }
                    const int ss = gseq / 9, tap = gseq - 9 * ss, rs = ss & 1;
                    if (!mbar_wait_warp(bar_raw_full + 8 * rs, (ss >> 1) & 1, abort_flag)) return false;
                    const int r = tap / 3, s = tap - 3 * r;
                    const int dr = P.tap_sign * (r - 1), dc = P.tap_sign * (s - 1);
                    const bool masked = (dc < 0 && edge_l) || (dc > 0 && edge_r);
                    const float *raw = (const float *)(raw_base + rs * (2 * L::RAW_BYTES)) + slab_pos + dr * P.img_w + dc;
#pragma unroll
                    for (int i = 0; i < BK; i++) av[i] = masked ? 0.f : raw[i * SLAB_PX];
                    if (gseq + 2 > 9 * ss + 8) {            // this group's last K-block of the slab
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_raw_empty + 8 * rs);
                    }
                    return true;
                } else if constexpr (ATMA) {
                    // this thread's row of K-block number gseq of the CTA's sequence: 32 values, one per channel, out of the raw
                    // tile TMA has delivered (chunk = warp of the group, pixel = lane: conflict-free 128-byte reads)
                    const int rs = gseq % RAWS;
                    if (!mbar_wait_warp(bar_raw_full + 8 * rs, (gseq / RAWS) & 1, abort_flag)) return false;
                    const float *raw = (const float *)(raw_base + rs * L::RAW_BYTES) + (warp & 3) * (BK * 32) + lane;
#pragma unroll
                    for (int i = 0; i < BK; i++) av[i] = raw[i * 32];
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_raw_empty + 8 * rs);       // this warp has read its chunk
                    return true;
                }
                const int mn = t % tiles_mn;
                if (mn != row_tile) {
                    row_tile = mn;
                    const int m = (mn % P.tiles_m) * BM + arow;
                    myRow = m < P.M_total ? __ldg(P.rowA + m) : make_int2(0, P.check == 1 ? 0 : (INVALID_Y << 16));
                    ry = myRow.y >> 16; rx = (int)(short)(myRow.y & 0xffff);
                }
                const int2 *kt = P.kA + (kb0 + it) * BK;
                const int4 *kc = (const int4 *)(P.kC + (kb0 + it) * BK);     // warp-uniform: four k entries per load
                const float *base = P.srcA + myRow.x;
                if (P.check == 0) {
                    // every tap of every row is inside the image (1x1 and other unpadded shapes)
#pragma unroll
                    for (int i = 0; i < BK / 4; i++) {
                        const int4 ke = __ldg(kc + i);
                        av[4 * i + 0] = __ldg(base + ke.x); av[4 * i + 1] = __ldg(base + ke.y);
                        av[4 * i + 2] = __ldg(base + ke.z); av[4 * i + 3] = __ldg(base + ke.w);
                    }
                } else if (P.check == 1) {
                    // myRow.y holds one bit per filter tap; the k entry holds (offset << 5) | tap number (31 = beyond K)
                    const unsigned taps = (unsigned)myRow.y;
#pragma unroll
                    for (int i = 0; i < BK / 4; i++) {
                        const int4 ke = __ldg(kc + i);
                        av[4 * i + 0] = (taps >> (ke.x & 31)) & 1u ? __ldg(base + (ke.x >> 5)) : 0.f;
                        av[4 * i + 1] = (taps >> (ke.y & 31)) & 1u ? __ldg(base + (ke.y >> 5)) : 0.f;
                        av[4 * i + 2] = (taps >> (ke.z & 31)) & 1u ? __ldg(base + (ke.z >> 5)) : 0.f;
                        av[4 * i + 3] = (taps >> (ke.w & 31)) & 1u ? __ldg(base + (ke.w >> 5)) : 0.f;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < BK; i++) {
                        const int2 ke = __ldg(kt + i);
                        const int y = ry + (ke.y >> 16), x = rx + (int)(short)(ke.y & 0xffff);
                        const bool ok = (unsigned)y < (unsigned)P.limY && (unsigned)x < (unsigned)P.limX;
                        av[i] = ok ? __ldg(base + ke.x) : 0.f;
                    }
                }
                return true;
            };
            auto store_row = [&](int s) {
                uint8_t *sA_hi = stage_base + s * L::STAGE_BYTES;
                uint8_t *sA_lo = sA_hi + L::A_BYTES;                      // only when SPLIT3
                if (CROSS_BF16) {
                    // plane 0: hi as TF32.  plane 1 (the cross-term operand, bf16, 64 values = one 128-byte row):
                    // columns 0-31 = lo(k), columns 32-63 = hi(k); the weight image holds [hi | lo], so one chain of
                    // bf16 MMAs over the 64 columns accumulates lo*hi + hi*lo.
#pragma unroll
                    for (int g = 0; g < BK / 8; g++) {
                        float hi[8], lo[8];
#pragma unroll
                        for (int j = 0; j < 8; j++) split_tf32(av[8 * g + j], hi[j], lo[j]);
                        *(float4 *)(sA_hi + swz(arow, g * 8)) = make_float4(hi[0], hi[1], hi[2], hi[3]);
                        *(float4 *)(sA_hi + swz(arow, g * 8 + 4)) = make_float4(hi[4], hi[5], hi[6], hi[7]);
                        *(uint4 *)(sA_lo + swz_chunk(arow, g)) =
                            make_uint4(pack_bf16(lo[0], lo[1]), pack_bf16(lo[2], lo[3]), pack_bf16(lo[4], lo[5]), pack_bf16(lo[6], lo[7]));
                        *(uint4 *)(sA_lo + swz_chunk(arow, 4 + g)) =
                            make_uint4(pack_bf16(hi[0], hi[1]), pack_bf16(hi[2], hi[3]), pack_bf16(hi[4], hi[5]), pack_bf16(hi[6], hi[7]));
                    }
                } else if (SPLIT3) {
#pragma unroll
                    for (int g = 0; g < BK / 4; g++) {
                        const uint32_t off = swz(arow, g * 4);
                        float4 hi, lo;
                        split_tf32(av[4 * g + 0], hi.x, lo.x); split_tf32(av[4 * g + 1], hi.y, lo.y);
                        split_tf32(av[4 * g + 2], hi.z, lo.z); split_tf32(av[4 * g + 3], hi.w, lo.w);
                        *(float4 *)(sA_hi + off) = hi; *(float4 *)(sA_lo + off) = lo;
                    }
                } else {
#pragma unroll
                    for (int g = 0; g < BK / 4; g++)
                        *(float4 *)(sA_hi + swz(arow, g * 4)) = make_float4(av[4 * g], av[4 * g + 1], av[4 * g + 2], av[4 * g + 3]);
                }
            };

            int t = blockIdx.x, kb0 = 0, nkb = 0, it = group;
            // carry `it` over tile boundaries until it names a K-block of tile t
            auto settle = [&]() {
                while (t < total_tiles) {
                    kb_range(t, kb0, nkb);
                    if (it < nkb) return;
                    it -= nkb; t += gridDim.x;
                }
            };
            settle();
            if (t < total_tiles && !load_row(t, kb0, it, group)) failed = true, fail_code = 6;
            for (int g = group; t < total_tiles && !failed; g += 2) {
                const int s = g % STAGES;
                const uint32_t par = ((g / STAGES) & 1) ^ 1;
                if (!mbar_wait_warp(bar_empty + 8 * s, par, abort_flag)) { failed = true, fail_code = 7; break; }
                if (arow == 0) {
                    // packed weights of this K-block / filter tile: one bulk copy into the stage's B_hi|B_lo area
                    const int n_tile = (t % tiles_mn) / P.tiles_m;
                    const uint32_t dstB = smem_u32(stage_base + s * L::STAGE_BYTES + (SPLIT3 ? 2 : 1) * L::A_BYTES);
                    const char *srcB = (const char *)P.packedB + ((size_t)(kb0 + it) * P.tiles_n + n_tile) * B_IMAGE;
                    mbar_expect_tx(bar_full + 8 * s, B_IMAGE);
                    tma_bulk_g2s(dstB, srcB, B_IMAGE, bar_full + 8 * s);
                }
                store_row(s);
                fence_async_smem();                 // generic-proxy stores -> visible to the tensor core (async proxy)
                __syncwarp();                       // orders the other lanes' stores and fences before lane 0's arrive
                if (lane == 0) mbar_arrive(bar_full + 8 * s);      // one arrive per warp: 32 lanes on one barrier word serialise
                if (tid == 0) *progress = g;        // paces the prefetch warp
                it += 2; settle();
                if (t < total_tiles && !load_row(t, kb0, it, g + 2)) failed = true, fail_code = 8;
            }
        } else {
            // backward-weight: one lane per k.  As above, two groups of four warps take alternate K-blocks; a warp gathers
            // 32 A rows and BN/4 B rows of its group's block.  A warp needs only ITS rows' table entries, so every warp keeps
            // a private copy of them in shared memory (written by its own lanes, read back as broadcasts): no warp waits on
            // another one here.
            constexpr int RA = BM / 4, RB = BN_ / 4;
            static_assert(RA == 32 && RB <= 32, "one table entry per lane");
            const int group = warp >> 2, wq = warp & 3;
            int2 *rowsA = (int2 *)(table_base + warp * (32 * 12));
            int *rowsB = (int *)(rowsA + 32);
            float av[RA], bv[BGATHER ? 1 : RB];
            // WGRAD with BGATHER: the dy operand (contiguous along k inside an image) is gathered with 16-byte loads, a
            // quarter warp per 128-byte row; the x operand (shifted by the filter taps) keeps one lane per k
            constexpr int BI = RB / 4;
            const int sub = lane >> 3, chunk = lane & 7;
            int offB[BGATHER ? BI : 1];
            float4 b4[BGATHER ? BI : 1];
            int row_tile = -1;
            auto load_tiles = [&](int mn, int kblock) {
                if (mn != row_tile) {
                    // new tile: refresh this warp's row entries (a warp-uniform branch)
                    row_tile = mn;
                    const int m0 = (mn % P.tiles_m) * BM, n0 = (mn / P.tiles_m) * BN_;
                    const int ma = m0 + wq * RA + lane, nb = n0 + wq * RB + lane;
                    __syncwarp();                       // every lane has finished reading the previous tile's entries
                    rowsA[lane] = ma < P.M_total ? __ldg(P.rowA + ma) : make_int2(0, INVALID_Y << 16);
                    if (!BGATHER) rowsB[lane] = (lane < RB && nb < P.N_total) ? __ldg(P.rowB + nb) : -1;
                    __syncwarp();
                    if constexpr (BGATHER) {
#pragma unroll
                        for (int i = 0; i < BI; i++) { const int n = n0 + wq * RB + 4 * i + sub; offB[i] = n < P.N_total ? __ldg(P.rowB + n) : 0; }
                    }
                }
                const int kbase = kblock * BK;
                const int2 ke = __ldg(P.kA + kbase + lane);
                const int ky = ke.y >> 16, kx = (int)(short)(ke.y & 0xffff);
                const float *base = P.srcA + ke.x;
#pragma unroll
                for (int r = 0; r < RA; r++) {
                    const int2 re = rowsA[r];
                    const int y = (re.y >> 16) + ky, x = (int)(short)(re.y & 0xffff) + kx;
                    const bool ok = (unsigned)y < (unsigned)P.limY && (unsigned)x < (unsigned)P.limX;
                    av[r] = ok ? __ldg(base + re.x) : 0.f;
                }
                if constexpr (BGATHER) {
                    const float *pb = P.srcB + __ldg(P.kB + kbase + chunk * 4);
#pragma unroll
                    for (int i = 0; i < BI; i++) b4[i] = ldg4(pb + offB[i]);
                } else {
                    const int kb = __ldg(P.kB + kbase + lane);
                    const float *bbase = P.srcB + (kb < 0 ? 0 : kb);
#pragma unroll
                    for (int r = 0; r < RB; r++) {
                        const int ro = rowsB[r];
                        bv[r] = (kb >= 0 && ro >= 0) ? __ldg(bbase + ro) : 0.f;
                    }
                }
            };
            auto store_tiles = [&](int s) {
                uint8_t *sA_hi = stage_base + s * L::STAGE_BYTES;
                uint8_t *sA_lo = sA_hi + L::A_BYTES;                      // only when SPLIT3
                uint8_t *sB_hi = sA_hi + (SPLIT3 ? 2 : 1) * L::A_BYTES;
                uint8_t *sB_lo = sB_hi + L::B_BYTES;
#pragma unroll
                for (int r = 0; r < RA; r++) {
                    const uint32_t off = swz(wq * RA + r, lane);
                    if (SPLIT3) { float hi, lo; split_tf32(av[r], hi, lo); *(float *)(sA_hi + off) = hi; *(float *)(sA_lo + off) = lo; }
                    else *(float *)(sA_hi + off) = av[r];
                }
                if constexpr (BGATHER) {
#pragma unroll
                    for (int i = 0; i < BI; i++) {
                        const uint32_t off = swz(wq * RB + 4 * i + sub, chunk * 4);
                        const float4 v = b4[i];
                        if (SPLIT3) {
                            float4 hi, lo;
                            split_tf32(v.x, hi.x, lo.x); split_tf32(v.y, hi.y, lo.y); split_tf32(v.z, hi.z, lo.z); split_tf32(v.w, hi.w, lo.w);
                            *(float4 *)(sB_hi + off) = hi; *(float4 *)(sB_lo + off) = lo;
                        } else {
                            *(float4 *)(sB_hi + off) = v;
                        }
                    }
                } else {
#pragma unroll
                    for (int r = 0; r < RB; r++) {
                        const uint32_t off = swz(wq * RB + r, lane);
                        if (SPLIT3) { float hi, lo; split_tf32(bv[r], hi, lo); *(float *)(sB_hi + off) = hi; *(float *)(sB_lo + off) = lo; }
                        else *(float *)(sB_hi + off) = bv[r];
                    }
                }
            };

            int t = blockIdx.x, kb0 = 0, nkb = 0, it = group;
            auto settle = [&]() {
                while (t < total_tiles) {
                    kb_range(t, kb0, nkb);
                    if (it < nkb) return;
                    it -= nkb; t += gridDim.x;
                }
            };
            settle();
            if (t < total_tiles) load_tiles(t % tiles_mn, kb0 + it);
            for (int g = group; t < total_tiles; g += 2) {
                const int s = g % STAGES;
                const uint32_t par = ((g / STAGES) & 1) ^ 1;
                if (!mbar_wait_warp(bar_empty + 8 * s, par, abort_flag)) { failed = true, fail_code = 9; break; }
                store_tiles(s);
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_full + 8 * s);
                it += 2; settle();
                if (t < total_tiles) load_tiles(t % tiles_mn, kb0 + it);
            }
        }
    } else if (warp == 8) {
        // ============================ MMA issuer (one thread) ============================
        // One thread feeds the tensor core, so its instruction stream is kept short: shared-memory descriptors differ only
        // in their 14-bit address field, which is advanced by adding constants (no field of the low word can carry into the
        // next: shared addresses stay below 256 KB), and stage / phase / accumulator rotation are running counters.
        if (lane == 0) {
            const uint32_t idesc = make_idesc(BN_);
            constexpr uint32_t DESC_HI = 64u | (1u << 14) | (2u << 29);       // upper word of make_desc()
            auto desc = [&](uint32_t lo) { return ((uint64_t)DESC_HI << 32) | lo; };
            const uint32_t stage0_lo = ((smem_u32(stage_base) >> 4) & 0x3FFFu) | (1u << 16);
            constexpr uint32_t STAGE_STEP = (uint32_t)L::STAGE_BYTES >> 4, A_STEP = (uint32_t)L::A_BYTES >> 4, B_STEP = (uint32_t)L::B_BYTES >> 4;
            int local = 0, set = 0;
            uint32_t s = 0, full_phase = 0, set_phase = 1, wh = 0;
            auto lo_word = [&](const uint8_t *ptr) { return ((smem_u32(ptr) >> 4) & 0x3FFFu) | (1u << 16); };
            const uint32_t w_hib_lo = lo_word(w_hib), w_lo_lo = lo_word(w_lo), w_x_lo = lo_word(w_x);
            const int nmain = P.nmain;
            for (int t = blockIdx.x; t < total_tiles && !failed; t += gridDim.x, local++) {
                int kb0, nkb; kb_range(t, kb0, nkb);
                if (!mbar_wait(bar_acc_empty + 8 * set, set_phase, abort_flag)) { failed = true, fail_code = 10; break; }
                tc_fence_after();
                const uint32_t set_base = tmem_base + (uint32_t)(set * set_cols);
                const uint32_t d_small = set_base + (uint32_t)small_off;
                int rot = 0;                   // which of the rotating main accumulators the next k-step adds into
                int fresh = nmain + 1;         // accumulators not written yet in this tile: the mains' first k-steps and the cross terms' first
                for (int it = 0; it < nkb; it++) {
                    if (!mbar_wait(bar_full + 8 * s, full_phase, abort_flag)) { failed = true, fail_code = 11; break; }
                    tc_fence_after();
                    uint32_t a_hi = stage0_lo + s * STAGE_STEP;
                    uint32_t a_lo = a_hi + A_STEP;
                    uint32_t b_hi = a_hi + (SPLIT3 ? 2u : 1u) * A_STEP;
                    uint32_t b_lo = b_hi + B_STEP;
                    if constexpr (WMODE) {
                        // s is the LO slot (0 / 1), wh the HI slot: hi planes where TMA put them, the rest in the LO slot
                        const uint32_t lo_slot = w_lo_lo + s * ((uint32_t)WL::LO_BYTES >> 4);
                        b_hi = w_hib_lo + wh * B_STEP;
                        if constexpr (WTMA) { a_hi = w_x_lo + wh * A_STEP; a_lo = lo_slot; b_lo = lo_slot + A_STEP; }
                        else { a_hi = lo_slot; a_lo = lo_slot + A_STEP; b_lo = lo_slot + (SPLIT3 ? 2u : 1u) * A_STEP; }
                    }
#pragma unroll
                    for (int ks = 0; ks < BK / 8; ks++) {
                        const uint32_t o = 2u * ks;      // 8 fp32 = 32 bytes along K inside the swizzle row = 2 units of 16 bytes
                        const bool first = (it == 0 && ks == 0);
                        if (SPLIT3) {
                            if (!CROSS_BF16) {
                                umma_tf32(d_small, desc(a_lo + o), desc(b_hi + o), idesc, first ? 0u : 1u);
                                umma_tf32(d_small, desc(a_hi + o), desc(b_lo + o), idesc, 1u);
                            } else {
                                // cross terms in bf16: 16 of the 64 [lo | hi] x [hi | lo] columns per instruction
                                umma_bf16(d_small, desc(a_lo + o), desc(b_lo + o), make_idesc_bf16(BN_), first ? 0u : 1u);
                            }
                        }
                        umma_tf32(set_base + (uint32_t)(rot * BN_), desc(a_hi + o), desc(b_hi + o), idesc, fresh > 1 ? 0u : 1u);
                        if (fresh > 1) fresh--;
                        if (++rot == nmain) rot = 0;
                    }
                    umma_commit(bar_empty + 8 * s);      // frees the stage (WMODE: the LO slot) when these MMAs have read it
                    if constexpr (WMODE) {
                        umma_commit(bar_raw_full + 8 * (HS + wh));      // ... and the HI slot
                        if (++wh == (uint32_t)HS) wh = 0;
                        if (++s == 2u) { s = 0; full_phase ^= 1u; }
                    } else if (++s == (uint32_t)STAGES) { s = 0; full_phase ^= 1u; }
                }
                if (!failed) umma_commit(bar_acc_full + 8 * set);     // this tile's accumulators are complete
                if (++set == nsets) { set = 0; set_phase ^= 1u; }
            }
        }
        __syncwarp();
    } else if (warp == 13) {
        // ============================ L2 prefetch of the A operand (warp 13) ============================
        // Layers with a short reduction and no padding (1x1) are bound by the latency of the producers' gather: a group
        // has one K-block (16 KB) in flight per round trip to HBM.  This warp walks the CTA's K-block sequence up to
        // PF_AHEAD blocks ahead of producer group 0 and touches one address per (pf_rows consecutive tile rows, k): the
        // rows are consecutive pixels, so that is every line the producers will read, and their loads then hit in L2.
        // Nothing waits on this warp; its own wait on the producers' progress is bounded and it simply stops on a time-out.
        if constexpr (WTMA) {
            // lane 0 fills the HI ring: for K-block number g of the CTA's sequence, 32 pixels of one image for the tile's 128
            // channel rows of x (A) and its BN filter rows of dy (B), as soon as the MMAs have released the slot
            if (lane == 0) {
                int g = 0;
                for (int t = blockIdx.x; t < total_tiles && !failed; t += gridDim.x) {
                    int kb0, nkb; kb_range(t, kb0, nkb);
                    const int mn = t % tiles_mn;
                    const int m0 = (mn % P.tiles_m) * BM, n0 = (mn / P.tiles_m) * BN_;
                    for (int it = 0; it < nkb; it++, g++) {
                        const int h = g % HS;
                        if (!mbar_wait(bar_raw_full + 8 * (HS + h), ((g / HS) & 1) ^ 1, abort_flag)) { failed = true, fail_code = 12; break; }
                        const int kbi = kb0 + it, img = kbi / P.chunks_per_image, x0 = (kbi % P.chunks_per_image) * 32;
                        mbar_expect_tx(bar_raw_full + 8 * h, (uint32_t)(WL::A_BYTES + WL::B_BYTES));
                        tma_load_3d(smem_u32(w_x + h * WL::X_BYTES), &P.mapA, x0, m0, img, bar_raw_full + 8 * h);
                        tma_load_3d(smem_u32(w_hib + h * WL::B_BYTES), &P.mapOut, x0, n0, img, bar_raw_full + 8 * h);
                    }
                }
            }
            __syncwarp();
        } else if constexpr (WSLAB) {
            // lane 0 fills the HI ring: per K-block the dy tile ([BN filters][32 pixels], swizzled: the hi plane of B) and the raw
            // slab of x ([16 channels][152 pixels] starting W + 1 pixels before the K-block, rounded down to 16 bytes)
            if (lane == 0) {
                int g = 0;
                const int W = P.img_w, cpi = P.chunks_per_image;
                for (int t = blockIdx.x; t < total_tiles && !failed; t += gridDim.x) {
                    int kb0, nkb; kb_range(t, kb0, nkb);
                    const int mn = t % tiles_mn;
                    const int c0 = (mn % P.tiles_m) * WS_CH, n0 = (mn / P.tiles_m) * BN_;
                    for (int it = 0; it < nkb; it++, g++) {
                        const int h = g % HS;
                        if (!mbar_wait(bar_raw_full + 8 * (HS + h), ((g / HS) & 1) ^ 1, abort_flag)) { failed = true, fail_code = 13; break; }
                        const int kbi = kb0 + it, img = kbi / cpi, x0 = (kbi % cpi) * 32;
                        const int base = ((x0 - W - 1 + 4096) & ~3) - 4096;
                        mbar_expect_tx(bar_raw_full + 8 * h, (uint32_t)(WL::B_BYTES + WL::X_BYTES));
                        tma_load_3d(smem_u32(w_hib + h * WL::B_BYTES), &P.mapOut, x0, n0, img, bar_raw_full + 8 * h);
                        tma_load_3d(smem_u32(w_x + h * WL::X_BYTES), &P.mapA, base, c0, img, bar_raw_full + 8 * h);
                    }
                }
            }
            __syncwarp();
        } else if constexpr (STMA) {
            // lane 0 feeds the slab ring: one box of [32 channels][SLAB_PX pixels] per (tile, channel group), two slabs deep
            if (lane == 0) {
                int ss = 0;
                const int tiles_per_image = P.chunks_per_image / 4;
                for (int t = blockIdx.x; t < total_tiles && !failed; t += gridDim.x) {
                    int kb0, nkb; kb_range(t, kb0, nkb);
                    const int tm = (t % tiles_mn) % P.tiles_m;
                    const int img = tm / tiles_per_image, t0 = (tm % tiles_per_image) * BM;
                    const int base = ((t0 - P.img_w - 1 + 4096) & ~3) - 4096;
                    for (int cg = 0; cg < nkb / 9; cg++, ss++) {
                        const int rs = ss & 1;
                        if (!mbar_wait(bar_raw_empty + 8 * rs, ((ss >> 1) & 1) ^ 1, abort_flag)) { failed = true, fail_code = 14; break; }
                        mbar_expect_tx(bar_raw_full + 8 * rs, (uint32_t)(2 * L::RAW_BYTES));
                        tma_load_3d(smem_u32(raw_base + rs * (2 * L::RAW_BYTES)), &P.mapA, base, (kb0 / 9 + cg) * BK, img, bar_raw_full + 8 * rs);
                    }
                }
            }
            __syncwarp();
        } else if constexpr (ATMA) {
            // ATMA: this warp's lane 0 feeds the raw activation ring: per K-block four boxes of [32 channels][32 pixels], one per
            // 32-pixel chunk of the tile's rows (a chunk lies inside one image; what lies past the image, the channels or the
            // batch arrives as zeros).  It runs RAWS K-blocks ahead of the producers across tile boundaries.
            if (lane == 0) {
                int g = 0;
                for (int t = blockIdx.x; t < total_tiles && !failed; t += gridDim.x) {
                    int kb0, nkb; kb_range(t, kb0, nkb);
                    const int cm0 = ((t % tiles_mn) % P.tiles_m) * (BM / 32);
                    int xs[4], zs[4];
#pragma unroll
                    for (int j = 0; j < 4; j++) { zs[j] = (cm0 + j) / P.chunks_per_image; xs[j] = ((cm0 + j) % P.chunks_per_image) * 32; }
                    for (int it = 0; it < nkb; it++, g++) {
                        const int rs = g % RAWS;
                        if (!mbar_wait(bar_raw_empty + 8 * rs, ((g / RAWS) & 1) ^ 1, abort_flag)) { failed = true, fail_code = 15; break; }
                        mbar_expect_tx(bar_raw_full + 8 * rs, (uint32_t)L::RAW_BYTES);
                        const uint32_t dst = smem_u32(raw_base + rs * L::RAW_BYTES);
#pragma unroll
                        for (int j = 0; j < 4; j++)
                            tma_load_3d(dst + j * (BK * 32 * 4), &P.mapA, xs[j], (kb0 + it) * BK, zs[j], bar_raw_full + 8 * rs);
                    }
                }
            }
            __syncwarp();
        } else if constexpr (A_ROWMAJOR && B_TMA) {
            if (P.pf_rows > 0) {
                const int nr = (BM + P.pf_rows - 1) / P.pf_rows;          // <= 32
                int g = 0;
                bool stop = false;
                for (int t = blockIdx.x; t < total_tiles && !stop; t += gridDim.x) {
                    int kb0, nkb; kb_range(t, kb0, nkb);
                    const int mn = t % tiles_mn;
                    const int m0 = (mn % P.tiles_m) * BM;
                    // lane j < nr: first row of group j; lane nr: the tile's last row (the line the last group spills into)
                    int mrow = lane < nr ? m0 + lane * P.pf_rows : m0 + BM - 1;
                    if (mrow >= P.M_total) mrow = P.M_total - 1;
                    const int roff = (lane <= nr && mrow >= m0) ? __ldg(P.rowA + mrow).x : -1;
                    for (int it = 0; it < nkb; it++, g++) {
                        // lane 0 paces the warp; its verdict is broadcast so that the shuffles below are reached by all lanes or none
                        int give_up = 0;
                        if (lane == 0) {
                            int spins = 0;
                            while (g > *progress + PF_AHEAD) {
                                if (*abort_flag || ++spins > (1 << 18)) { give_up = 1; break; }
                                __nanosleep(128);
                            }
                        }
                        give_up = __shfl_sync(0xffffffffu, give_up, 0);
                        if (give_up) { stop = true; break; }
                        const float *pk = P.srcA + __ldg(P.kC + (kb0 + it) * BK + lane);
                        for (int j = 0; j <= nr && j < 32; j++) {
                            const int ro = __shfl_sync(0xffffffffu, roff, j);
                            if (ro >= 0) asm volatile("prefetch.global.L2 [%0];" ::"l"(pk + ro));
                        }
                    }
                }
            }
        }
    } else {
        // ============================ epilogue (warps 9-12) ============================
        const int quarter = warp & 3;                     // the TMEM lane quarter this warp may access
        int local = 0;
        for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, local++) {
            const int mn = t % tiles_mn, split = t / tiles_mn;
            const int m0 = (mn % P.tiles_m) * BM, n0 = (mn / P.tiles_m) * BN_;
            const int set = local % nsets;
            if (!mbar_wait_warp(bar_acc_full + 8 * set, (local / nsets) & 1, abort_flag)) { failed = true, fail_code = 16; break; }
            tc_fence_after();
            if constexpr (ATMA) {
                // This warp's 32 rows are one 32-pixel chunk of one image.  Per 32 columns: drain the accumulators, write the
                // [32 columns][32 pixels] block into one of the warp's two staging buffers (lane = pixel: conflict-free), and
                // let TMA store it -- or add it -- into out[image][n0 + 32c ...][x0 ...]; pixels past the end of the image and
                // columns past the last filter are dropped by the copy.
                const int cm = m0 / 32 + quarter;
                const int img = cm / P.chunks_per_image, x0 = (cm % P.chunks_per_image) * 32;
                const uint32_t set_base = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(set * set_cols);
                // two warps share a lane quarter: warps 9-12 take the even 32-column chunks, warps 14-17 the odd ones
                const int half = warp >= 14 ? 1 : 0;
                constexpr int NCHUNK = (BN_ + 31) / 32;
                float *sb = (float *)(out_base + (half * 4 + quarter) * (32 * 32 * 4));
                if (half >= NCHUNK) {                       // BN = 32: nothing for the second set to drain
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_acc_empty + 8 * set);
                    continue;
                }
#pragma unroll 1
                for (int c = half; c < NCHUNK; c += 2) {
                    uint32_t r[32], tt[32];
                    tmem_ld32(set_base + (uint32_t)(c * 32), r);
#pragma unroll 1
                    for (int a = 1; a < nacc; a++) {
                        tmem_ld32(set_base + (uint32_t)(a * BN_ + c * 32), tt);
#pragma unroll
                        for (int j = 0; j < 32; j++) r[j] = __float_as_uint(__fadd_rn(__uint_as_float(r[j]), __uint_as_float(tt[j])));
                    }
                    if (c + 2 >= NCHUNK) {                  // this warp's last chunk of the set
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_acc_empty + 8 * set);
                    }
                    const int col0 = n0 + c * 32;
                    if (col0 < P.N_total && img < P.images) {             // warp-uniform
                        // the copy that last used this warp's staging buffer must have read it (it had the whole
                        // tensor-memory round trip above to do so)
                        if (lane == 0) tma_wait_group_read<0>();
                        __syncwarp();
                        if (P.bias) {
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                sb[j * 32 + lane] = __fadd_rn(__uint_as_float(r[j]), col0 + j < P.N_total ? __ldg(P.bias + col0 + j) : 0.f);
                        } else if (P.add_zero) {
#pragma unroll
                            for (int j = 0; j < 32; j++) sb[j * 32 + lane] = __fadd_rn(0.f, __uint_as_float(r[j]));
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j++) sb[j * 32 + lane] = __uint_as_float(r[j]);
                        }
                        fence_async_smem();                 // generic-proxy stores -> visible to the copy engine
                        __syncwarp();
                        if (lane == 0) {
                            if (P.reduce_out) tma_reduce_add_3d(&P.mapOut, x0, col0, img, smem_u32(sb));
                            else tma_store_3d(&P.mapOut, x0, col0, img, smem_u32(sb));
                            tma_commit_group();
                        }
                    }
                }
                continue;
            }
            const int m = m0 + quarter * 32 + lane;
            // WSLAB: row r of tile tm is element tm * 126 + r of the (channel, tap) space (rows 126 and 127 hold nothing)
            const int ws_off = (m0 / BM) * WS_ROWS + quarter * 32 + lane;
            const bool m_ok = WSLAB ? (quarter * 32 + lane < WS_ROWS && ws_off < P.M_total) : m < P.M_total;
            float *obase = P.out + (long long)split * P.split_stride + (m_ok ? (WSLAB ? (long long)ws_off : (long long)__ldg(P.outM + m)) : 0);
            if (P.accumulate && !WSLAB) {
                // The read-modify-write below waits on the old output values.  While this tile's MMAs are still running,
                // pull the lines of the NEXT tile of this CTA into L2 (the first tile prefetches its own): lane j of the
                // warp takes columns j, j + 32, ... of the warp's 32 rows (one 128-byte line each).
                const int tn = (local == 0) ? t : t + (int)gridDim.x;
                if (tn < total_tiles) {
                    const int mn2 = tn % tiles_mn;
                    const int mrow = (mn2 % P.tiles_m) * BM + quarter * 32, ncol0 = (mn2 / P.tiles_m) * BN_;
                    if (mrow < P.M_total) {
                        const float *line = P.out + (long long)(tn / tiles_mn) * P.split_stride + (long long)__ldg(P.outM + mrow);
#pragma unroll
                        for (int j = lane; j < BN_; j += 32)
                            if (ncol0 + j < P.N_total)
                                asm volatile("prefetch.global.L2 [%0];" ::"l"(line + (long long)(ncol0 + j) * P.out_n_stride));
                    }
                }
            }
            const uint32_t set_base = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(set * set_cols);
#pragma unroll 1
            for (int c = 0; c < (BN_ + 31) / 32; c++) {
                uint32_t r[32], tt[32];
                float *p = obase + (long long)(n0 + c * 32) * P.out_n_stride;
                const long long stride = P.out_n_stride;
                const int ncols = P.N_total - (n0 + c * 32);           // columns of this chunk inside the problem
                // read-modify-write: the 32 loads of the old values go out first and overlap the tensor-memory reads
                float prev[32];
                const bool rmw = P.accumulate && m_ok && ncols >= 32;
                if (rmw) {
                    const float *q = p;
#pragma unroll
                    for (int j = 0; j < 32; j++) { prev[j] = __ldcg(q); q += stride; }
                }
                tmem_ld32(set_base + (uint32_t)(c * 32), r);
                // every accumulator in use holds data: a tile has at least four k-steps
#pragma unroll 1
                for (int a = 1; a < nacc; a++) {
                    tmem_ld32(set_base + (uint32_t)(a * BN_ + c * 32), tt);
#pragma unroll
                    for (int j = 0; j < 32; j++) r[j] = __float_as_uint(__fadd_rn(__uint_as_float(r[j]), __uint_as_float(tt[j])));
                }
                if (c == (BN_ + 31) / 32 - 1) {
                    // all of this set has been read: hand it back to the MMA warp before the global stores
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_acc_empty + 8 * set);
                }
                if (m_ok) {
                    // The four epilogue warps are a serial instruction stream per tile, so the store loop is kept free of
                    // branches and index arithmetic: full 32-column chunks take a straight-line path with a running pointer.
                    if (ncols >= 32) {
                        if (rmw) {
#pragma unroll
                            for (int j = 0; j < 32; j++) { *p = __fadd_rn(prev[j], __uint_as_float(r[j])); p += stride; }
                        } else if (P.bias) {
                            const float *bq = P.bias + n0 + c * 32;
                            float bj[32];
#pragma unroll
                            for (int j = 0; j < 32; j++) bj[j] = __ldg(bq + j);
#pragma unroll
                            for (int j = 0; j < 32; j++) { *p = __fadd_rn(__uint_as_float(r[j]), bj[j]); p += stride; }
                        } else if (P.add_zero) {
#pragma unroll
                            for (int j = 0; j < 32; j++) { *p = __fadd_rn(0.f, __uint_as_float(r[j])); p += stride; }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j++) { *p = __uint_as_float(r[j]); p += stride; }
                        }
                    } else {
#pragma unroll 1
                        for (int j = 0; j < ncols; j++) {
                            // r[] must stay in registers: select the j-th value without dynamic indexing
                            float v = 0.f;
#pragma unroll
                            for (int i = 0; i < 32; i++) if (i == j) v = __uint_as_float(r[i]);
                            if (P.accumulate) v = __fadd_rn(__ldcg(p), v);
                            else if (P.bias) v = __fadd_rn(v, __ldg(P.bias + n0 + c * 32 + j));
                            else if (P.add_zero) v = __fadd_rn(0.f, v);
                            *p = v; p += stride;
                        }
                    }
                }
            }
        }
        if constexpr (ATMA) {
            // the staging buffers must outlive the copies that read them
            if (lane == 0) tma_wait_group<0>();
            __syncwarp();
        }
    }
    // status word: site of the first wait that gave up | warp << 8 | kernel variant (TMA mode << 16, WGRAD << 20, BGATHER << 21)
    if (failed) { *abort_flag = 1; atomicCAS(P.status, 0, fail_code | (warp << 8) | (TMA << 16) | ((WGRAD ? 1 : 0) << 20) | ((BGATHER ? 1 : 0) << 21)); }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) tmem_dealloc(tmem_base, 512);
}

// ---- index tables ----------------------------------------------------------------------------------
__device__ __forceinline__ int pack_yx(int y, int x) { return (y << 16) | (x & 0xffff); }

struct TableArgs {
    ConvGeom g; int mode;       // 0 fwd, 1 bwd-data, 2 bwd-weight
    // backward-data only: residue class (ca, cb) of (y+pt, x+pl) modulo the strides.  Input pixels of one
    // class receive contributions only from the taps r = ca + r'*sr, s = cb + s'*sc, which turns a strided
    // backward pass into sr*sc dense stride-1 problems with no wasted taps.
    int ca, cb, y0, x0, hc, wc, rt, st_;
    int check, limY, limX;   // check == 1: rowA.y = bitmask over taps, kA.y = tap number
    int2 *rowA, *kA; int *rowB, *kB, *outM, *kC;
    int M_total, N_total, K_total, K_pad;
};

__global__ void __launch_bounds__(256) build_tables_kernel(TableArgs T) {
    const ConvGeom g = T.g;
    const int pq = g.oh * g.ow, hw = g.ih * g.iw, rs = g.kr * g.kc;
    const long long total = (long long)T.M_total + T.K_pad + T.N_total;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        if (i < T.M_total) {
            const int m = (int)i;
            if (T.mode == 0) {              // output pixel
                const int n = m / pq, t = m - n * pq, p = t / g.ow, q = t - p * g.ow;
                const int y = p * g.sr - g.pt, x = q * g.sc - g.pl;
                int tag = pack_yx(y, x);
                if (T.check == 1) {
                    tag = 0;
                    for (int r = 0; r < g.kr; r++) for (int s2 = 0; s2 < g.kc; s2++)
                        if ((unsigned)(y + r) < (unsigned)T.limY && (unsigned)(x + s2) < (unsigned)T.limX) tag |= 1 << (r * g.kc + s2);
                }
                T.rowA[m] = make_int2(n * g.c * hw + y * g.iw + x, tag);
                T.outM[m] = n * g.k * pq + t;
            } else if (T.mode == 1) {       // input pixel of the residue class
                const int per = T.hc * T.wc;
                const int n = m / per, t = m - n * per, i = t / T.wc, j = t - i * T.wc;
                const int y = T.y0 + i * g.sr, x = T.x0 + j * g.sc;
                const int yc = (y + g.pt - T.ca) / g.sr, xc = (x + g.pl - T.cb) / g.sc;
                int tag = pack_yx(yc, xc);
                if (T.check == 1) {
                    tag = 0;
                    for (int r2 = 0; r2 < T.rt; r2++) for (int s2 = 0; s2 < T.st_; s2++)
                        if ((unsigned)(yc - r2) < (unsigned)T.limY && (unsigned)(xc - s2) < (unsigned)T.limX) tag |= 1 << (r2 * T.st_ + s2);
                }
                T.rowA[m] = make_int2(n * g.k * pq + yc * g.ow + xc, tag);
                T.outM[m] = n * g.c * hw + y * g.iw + x;
            } else if (T.mode == 3) {       // output pixel of dy; result column plane T[n][(c,r,s)][p][q]
                const int n = m / pq, t = m - n * pq;
                T.rowA[m] = make_int2(n * g.k * pq + t, pack_yx(0, 0));
                T.outM[m] = n * g.c * rs * pq + t;
            } else if (T.mode == 4) {       // plain GEMM C[M x N] = op(A) op(B): g.n = M, g.c = K, g.k = N, g.ih / g.iw = transpose flags
                T.rowA[m] = make_int2(g.ih ? m : m * g.c, pack_yx(0, 0));
                T.outM[m] = m * g.k;
            } else {                        // (c, r, s)
                const int c = m / rs, t = m - c * rs, r = t / g.kc, s = t - r * g.kc;
                T.rowA[m] = make_int2(c * hw + (r - g.pt) * g.iw + (s - g.pl), pack_yx(r - g.pt, s - g.pl));
                T.outM[m] = m;
            }
        } else if (i < (long long)T.M_total + T.K_pad) {
            const int k = (int)(i - T.M_total);
            if (T.check == 5) {
                // slab-fed 3x3 kernels: k = (32-channel group, tap, channel in group); only the weight offsets are needed
                const int cg = k / (9 * BK), rem = k - cg * 9 * BK, tap = rem / BK, ch = cg * BK + (rem - tap * BK);
                const int nch = T.mode == 0 ? g.c : g.k;
                T.kA[k] = make_int2(0, 0); T.kC[k] = 0;
                T.kB[k] = ch >= nch ? -1 : (T.mode == 0 ? ch * rs + tap : ch * g.c * rs + tap);
                continue;
            }
            if (k >= T.K_total) { T.kA[k] = make_int2(0, T.check == 1 ? 31 : pack_yx(INVALID_Y, 0)); T.kC[k] = 31; T.kB[k] = -1; continue; }
            if (T.mode == 0) {              // (c, r, s)
                const int c = k / rs, t = k - c * rs, r = t / g.kc, s = t - r * g.kc;
                T.kA[k] = make_int2(c * hw + r * g.iw + s, T.check == 1 ? t : pack_yx(r, s));
                T.kB[k] = k;
            } else if (T.mode == 1) {       // (f, r', s') with r = ca + r'*sr, s = cb + s'*sc
                const int taps = T.rt * T.st_;
                const int f = k / taps, t = k - f * taps, r2 = t / T.st_, s2 = t - r2 * T.st_;
                T.kA[k] = make_int2(f * pq - r2 * g.ow - s2, T.check == 1 ? t : pack_yx(-r2, -s2));
                T.kB[k] = f * g.c * rs + (T.ca + r2 * g.sr) * g.kc + (T.cb + s2 * g.sc);
            } else if (T.mode == 3) {       // filter f
                T.kA[k] = make_int2(k * pq, pack_yx(0, 0));
                T.kB[k] = k * g.c * rs;
            } else if (T.mode == 4) {       // op(A)[m][k] = A[k * M + m] or A[m * K + k];  op(B)[k][n] = B[n * K + k] or B[k * N + n]
                T.kA[k] = make_int2(g.ih ? k * g.n : k, pack_yx(0, 0));
                T.kB[k] = g.iw ? k : k * g.k;
            } else {                        // (n, p, q)
                const int n = k / pq, t = k - n * pq, p = t / g.ow, q = t - p * g.ow;
                T.kA[k] = make_int2(n * g.c * hw + p * g.sr * g.iw + q * g.sc, pack_yx(p * g.sr, q * g.sc));
                T.kB[k] = n * g.k * pq + t;
            }
            const int2 ka = T.kA[k];
            T.kC[k] = T.check == 0 ? ka.x : T.check == 1 ? (int)(((unsigned)ka.x << 5) | (unsigned)ka.y) : 0;
        } else {
            const int n = (int)(i - T.M_total - T.K_pad);
            if (T.mode == 0) T.rowB[n] = n * g.c * rs;          // filter row of w[f][c*r*s]
            else if (T.mode == 1) T.rowB[n] = n * rs;           // in-channel c of w[f][c][r][s]
            else if (T.mode == 3) T.rowB[n] = n;                // (c,r,s) column of w[f][c*r*s]
            else if (T.mode == 4) T.rowB[n] = g.iw ? n * g.c : n;
            else T.rowB[n] = n * pq;                            // filter plane of dy[n][f][p*q]
        }
    }
}

// B operand of forward / backward-data (the weights), prepared once per call: for every (K-block, filter tile) the
// [BN x 32] tile is written in the exact shared-memory image the MMA reads (K-major SWIZZLE_128B), hi plane then lo
// plane, so the main kernel fetches it with a single 16-byte-aligned TMA bulk copy.  The tile is read with consecutive
// threads along the dimension that is contiguous in the weight tensor -- k for forward (w[f][c*r*s]), the in-channel row
// for backward-data (w[f][c][r][s] with k = (f, r, s)) -- staged in shared memory, and written out 16 bytes per thread.
__device__ __forceinline__ void pack_b_tile(const float *__restrict__ src, const int *__restrict__ rowB, const int *__restrict__ kB,
                                            float *__restrict__ packed, int bn, int n_total, int tiles_n, int row_fastest, int prec, int kb, int nt,
                                            float (*tile)[BK + 1]) {
    const bool split3 = prec != 1;
    const size_t image_floats = (size_t)bn * BK * (split3 ? 2 : 1);
    char *img = (char *)(packed + ((size_t)kb * tiles_n + nt) * image_floats);
    // blockDim.x = 256 is a multiple of BK and of bn, so one of the two coordinates is fixed per thread: its table entry is
    // looked up once, and the loop's loads are independent of each other (several in flight per thread)
    if (row_fastest) {
        const int row = threadIdx.x % bn, n = nt * bn + row;
        const int ro = n < n_total ? __ldg(rowB + n) : -1;
#pragma unroll 4
        for (int k = threadIdx.x / bn; k < BK; k += 256 / bn) {
            const int ko = __ldg(kB + kb * BK + k);
            tile[row][k] = (ro >= 0 && ko >= 0) ? __ldg(src + ro + ko) : 0.f;
        }
    } else {
        const int k = threadIdx.x % BK;
        const int ko = __ldg(kB + kb * BK + k);
#pragma unroll 4
        for (int row = threadIdx.x / BK; row < bn; row += 256 / BK) {
            const int n = nt * bn + row;
            tile[row][k] = (n < n_total && ko >= 0) ? __ldg(src + __ldg(rowB + n) + ko) : 0.f;
        }
    }
    __syncthreads();
    char *plane1 = img + (size_t)bn * BK * 4;
    for (int q = threadIdx.x; q < bn * (BK / 4); q += blockDim.x) {
        const int row = q / (BK / 4), c = q % (BK / 4);
        const float4 v = make_float4(tile[row][4 * c], tile[row][4 * c + 1], tile[row][4 * c + 2], tile[row][4 * c + 3]);
        const uint32_t off = swz(row, 4 * c);
        if (split3) {
            float4 hi, lo;
            split_tf32(v.x, hi.x, lo.x); split_tf32(v.y, hi.y, lo.y); split_tf32(v.z, hi.z, lo.z); split_tf32(v.w, hi.w, lo.w);
            *(float4 *)(img + off) = hi;
            if (prec == 0) *(float4 *)(plane1 + off) = lo;
        } else {
            *(float4 *)(img + off) = v;
        }
    }
    if (prec == 2) {
        // plane 1: bf16 row of 64 = [hi(0..31) | lo(0..31)], the partner of the A rows' [lo | hi]; one 16-byte chunk = 8 values
        for (int q = threadIdx.x; q < bn * 8; q += blockDim.x) {
            const int row = q / 8, c = q % 8, k0 = (c & 3) * 8;
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float h0, l0, h1, l1;
                split_tf32(tile[row][k0 + 2 * j], h0, l0); split_tf32(tile[row][k0 + 2 * j + 1], h1, l1);
                w[j] = c < 4 ? pack_bf16(h0, h1) : pack_bf16(l0, l1);
            }
            *(uint4 *)(plane1 + swz_chunk(row, c)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
}

__global__ void __launch_bounds__(256) pack_b_kernel(const float *__restrict__ src, const int *__restrict__ rowB, const int *__restrict__ kB,
                                                     float *__restrict__ packed, int bn, int n_total, int tiles_n, int row_fastest, int prec) {
    __shared__ float tile[128][BK + 1];
    pack_b_tile(src, rowB, kB, packed, bn, n_total, tiles_n, row_fastest, prec, blockIdx.x, blockIdx.y, tile);
}

// Many weight tensors in ONE launch.  The weights of a net change once per step (the optimizer), while every layer needs
// them packed twice (the forward and the backward-data tilings): the packed images are kept per (tensor, tiling), and the
// first convolution call that finds its image out of date re-packs every image that is out of date with this kernel.
struct PackJob { const float *src; const int *rowB, *kB; float *dst; int bn, n_total, tiles_n, row_fastest, prec, kblocks; };
constexpr int kMaxPackJobs = 256;
struct MultiPackArgs { const PackJob *jobs; int n; unsigned short slot[kMaxPackJobs]; unsigned start[kMaxPackJobs + 1]; };

__global__ void __launch_bounds__(256) pack_b_multi_kernel(const __grid_constant__ MultiPackArgs A) {
    __shared__ float tile[128][BK + 1];
    // which job does this block belong to: the last one whose first block is <= blockIdx.x
    int lo = 0, hi = A.n - 1;
    while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (A.start[mid] <= blockIdx.x) lo = mid; else hi = mid - 1; }
    const PackJob j = A.jobs[A.slot[lo]];
    const unsigned local = blockIdx.x - A.start[lo];
    pack_b_tile(j.src, j.rowB, j.kB, j.dst, j.bn, j.n_total, j.tiles_n, j.row_fastest, j.prec, (int)(local / j.tiles_n), (int)(local % j.tiles_n), tile);
}

template <int BN_, int PREC, bool WGRAD, bool BGATHER = false, int TMA = 0>
int launch_variant(DevCtx *cx, cudaStream_t st, const TcParams &P, dim3 grid, int dev) {
    using L = Layout<BN_, PREC != 1, TMA == 1 || TMA == 3, TMA == 4>;
    constexpr int SMEM = (TMA == 2 || TMA == 4) ? WLayout<BN_, PREC != 1, TMA == 4>::SMEM_BYTES : L::SMEM_BYTES;
    static bool configured_dev[EDDLB200_MAX_DEVICES] = {};
    bool &configured = configured_dev[dev];
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(igemm_tc_kernel<BN_, PREC, WGRAD, BGATHER, TMA>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return cuda_status(e, "conv_tc(smem attribute)");
        configured = true;
    }
    igemm_tc_kernel<BN_, PREC, WGRAD, BGATHER, TMA><<<grid, threads_of(TMA), SMEM, st>>>(P);
    EB_LAUNCH_CHECK("conv_tc");
    return 0;
}

template <int PREC, bool WGRAD, bool BGATHER = false, int TMA = 0>
int launch_bn(DevCtx *cx, cudaStream_t st, const TcParams &P, dim3 grid, int bn, int dev) {
    if (bn == 32) return launch_variant<32, PREC, WGRAD, BGATHER, TMA>(cx, st, P, grid, dev);
    if (bn == 64) return launch_variant<64, PREC, WGRAD, BGATHER, TMA>(cx, st, P, grid, dev);
    return launch_variant<128, PREC, WGRAD, BGATHER, TMA>(cx, st, P, grid, dev);
}

// [images][channels][pixels] fp32 tensor as a 3-D tensor map with boxes of 32 pixels x 32 channels of one image, no swizzle:
// the box lands in shared memory as [32 channels][32 pixels].  Needs a 16-byte aligned base and pixels % 4 == 0.
// With swizzle128 the box (box_rows channels x 32 pixels = box_rows rows of 128 bytes) lands in the K-major SWIZZLE_128B layout
// of an MMA operand whose k runs along the pixels.
bool encode_plane_map(CUtensorMap *map, const float *base, int pixels, int channels, int images, int box_rows = 32, bool swizzle128 = false, int box_px = 32) {
    const cuuint64_t dims[3] = {(cuuint64_t)pixels, (cuuint64_t)channels, (cuuint64_t)images};
    const cuuint64_t strides[2] = {(cuuint64_t)pixels * 4, (cuuint64_t)pixels * channels * 4};
    const cuuint32_t box[3] = {(cuuint32_t)box_px, (cuuint32_t)box_rows, 1}, elem[3] = {1, 1, 1};
    // the driver entry point is looked up at run time: the library must load (and refuse work) on a machine without a driver
    typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                 const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    static bool looked_up = false;
    if (!looked_up) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) encode = (EncodeFn)fn;
        else cudaGetLastError();
        looked_up = true;
    }
    if (!encode) return false;
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float *>(base), dims, strides, box, elem,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
int g_conv_tma = 2;            // eddlb200_set_option("conv_tma", 0 off / 1 stores only / 2 stores and adds)
int g_conv_tma3 = 1;           // eddlb200_set_option("conv_tma_3x3", 0 / 1)
int g_conv_wslab = 1;          // eddlb200_set_option("conv_tma_wgrad_3x3", 0 / 1)
int g_conv_wtma = 2;           // eddlb200_set_option("conv_tma_wgrad", 0 off / 1 on / 2 on, landed values used as the hi plane as they are)

int *g_status[EDDLB200_MAX_DEVICES] = {};
int g_conv_prefetch = 1;       // eddlb200_set_option("conv_prefetch", 0 / 1)

// The index tables are a pure function of the problem geometry, so they are built once per distinct geometry and kept
// in device memory (a few MB per ResNet-50 layer shape); past the budget, tables go to the scratch arena and are
// rebuilt every call.
struct TableCache {
    std::mutex mu;
    std::map<std::array<int, 24>, char *> entries;
    size_t bytes = 0;
};
TableCache g_tables[EDDLB200_MAX_DEVICES];
constexpr size_t kTableCacheBudget = size_t(1) << 30;

std::array<int, 24> table_key(const TableArgs &T) {
    const ConvGeom &g = T.g;
    return {T.mode, g.n, g.c, g.ih, g.iw, g.k, g.kr, g.kc, g.oh, g.ow, g.sr, g.sc, g.pt, g.pl,
            T.ca, T.cb, T.y0, T.x0, T.hc, T.wc, T.rt, T.st_, T.check, T.K_pad};
}

// Packed weight images, one per (weight tensor, tiling), valid while the tensor's write-observer version stands.
struct PackEntry {
    std::array<int, 24> tkey; int bn, precision; const float *src; size_t src_bytes;
    float *packed; size_t packed_bytes;
    unsigned blocks;                       // K-blocks x filter tiles = thread blocks that pack it
    unsigned long long version;            // version of src the image was made from (0 = never)
};
struct PackCache {
    std::mutex mu;
    std::vector<PackEntry> entries;        // slot = index, also the index into the device job table
    PackJob *jobs = nullptr;               // device memory, kMaxPackJobs entries
};
PackCache g_packs[EDDLB200_MAX_DEVICES];
int g_conv_pack_cache = 1;                 // eddlb200_set_option("conv_pack_cache", 0 / 1)

// The packed image of `src` for this tiling, re-packing every out-of-date image of the device in one launch when this
// one is out of date.  nullptr = not cached (the caller packs into scratch for this call).  rowB / kB must be cached tables.
const float *packed_weights(DevCtx *cx, cudaStream_t st, int dev, const std::array<int, 24> &tkey, int bn, int precision, const float *src,
                            size_t src_bytes, const int *rowB, const int *kB, int kblocks, int tiles_n, int n_total, int row_fastest) {
    if (!g_conv_pack_cache) return nullptr;
    PackCache &pc = g_packs[dev];
    std::lock_guard<std::mutex> lock(pc.mu);
    if (!pc.jobs && cudaMalloc((void **)&pc.jobs, sizeof(PackJob) * kMaxPackJobs) != cudaSuccess) { cudaGetLastError(); pc.jobs = nullptr; return nullptr; }
    int slot = -1;
    for (size_t i = 0; i < pc.entries.size(); i++) {
        const PackEntry &e = pc.entries[i];
        if (e.src == src && e.bn == bn && e.precision == precision && e.tkey == tkey) { slot = (int)i; break; }
    }
    const size_t packed_bytes = (size_t)kblocks * tiles_n * bn * BK * sizeof(float) * (precision != 1 ? 2 : 1);
    if (slot < 0) {
        // a new image: take a free slot, or the slot of an image whose tensor is gone (released memory is no longer observed)
        if ((int)pc.entries.size() < kMaxPackJobs) { pc.entries.push_back(PackEntry{}); slot = (int)pc.entries.size() - 1; }
        else {
            for (size_t i = 0; i < pc.entries.size() && slot < 0; i++)
                if (watch_version(cx, pc.entries[i].src) == 0) slot = (int)i;
            if (slot < 0) return nullptr;
            cudaStreamSynchronize(st);                  // kernels already enqueued may still read the old image
            cudaFree(pc.entries[slot].packed);
            pc.entries[slot] = PackEntry{};
        }
        PackEntry &e = pc.entries[slot];
        if (cudaMalloc((void **)&e.packed, packed_bytes) != cudaSuccess) { cudaGetLastError(); e = PackEntry{}; return nullptr; }
        e.tkey = tkey; e.bn = bn; e.precision = precision; e.src = src; e.src_bytes = src_bytes; e.packed_bytes = packed_bytes;
        e.blocks = (unsigned)kblocks * (unsigned)tiles_n; e.version = 0;
        const PackJob job{src, rowB, kB, e.packed, bn, n_total, tiles_n, row_fastest, precision, kblocks};
        // pageable source: staged before the call returns
        if (cudaMemcpyAsync(pc.jobs + slot, &job, sizeof(job), cudaMemcpyHostToDevice, st) != cudaSuccess) { cudaGetLastError(); cudaFree(e.packed); e = PackEntry{}; return nullptr; }
    }
    PackEntry &me = pc.entries[slot];
    const unsigned long long now = watch_add(cx, src, src_bytes);         // registers the tensor on first use
    if (me.version != 0 && me.version == now) return me.packed;
    // out of date: this image and every other one whose tensor has been written since it was packed
    MultiPackArgs A;
    A.jobs = pc.jobs; A.n = 0;
    unsigned total = 0;
    std::vector<unsigned long long> seen(pc.entries.size(), 0);
    for (size_t i = 0; i < pc.entries.size(); i++) {
        PackEntry &e = pc.entries[i];
        if (!e.packed) continue;
        const unsigned long long v = (int)i == slot ? now : watch_version(cx, e.src);
        if (v == 0 || v == e.version) continue;         // tensor no longer observed (released), or image up to date
        A.slot[A.n] = (unsigned short)i; A.start[A.n] = total; total += e.blocks; seen[i] = v; A.n++;
    }
    A.start[A.n] = total;
    pack_b_multi_kernel<<<total, 256, 0, st>>>(A);
    count_launch(cx);
    if (cudaGetLastError() != cudaSuccess) return nullptr;
    for (int i = 0; i < A.n; i++) pc.entries[A.slot[i]].version = seen[A.slot[i]];
    return me.packed;
}

// out[i] = sum_s part[s][i] (+ bias[(i / plane) % nbias])      (split-K forward)
__global__ void __launch_bounds__(256) splitk_store_kernel(const float *__restrict__ part, float *__restrict__ out, size_t count, int splits,
                                                           const float *__restrict__ bias, int plane, int nbias) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        float v = 0.f;
        for (int z = 0; z < splits; z++) v += part[(size_t)z * count + i];
        if (bias) v = __fadd_rn(v, __ldg(bias + (i / plane) % nbias));
        out[i] = v;
    }
}

// One GEMM launch (tables + main kernel + optional split-K combine).  T carries mode / class fields and the
// problem extents; out_total is the element count of the output tensor (the unit of a split-K partial).
int run_one(DevCtx *cx, cudaStream_t st, int dev, TableArgs T, TcParams P, const float *srcA, const float *srcB, float *out,
            const float *bias, int precision, size_t out_total, bool allow_split, bool out_zero = false) {
    const ConvGeom &g = T.g;
    const int mode = T.mode;
    T.K_pad = (T.K_total + BK - 1) / BK * BK;
    // how the gathered operand is tested against the zero padding
    T.limY = P.limY; T.limX = P.limX;
    T.check = 2;
    if (mode == 3 || mode == 4) T.check = (T.K_total % BK == 0) ? 0 : 2;
    else if (mode == 0) {
        const bool inside = g.pt == 0 && g.pl == 0 && (g.oh - 1) * g.sr + g.kr <= g.ih && (g.ow - 1) * g.sc + g.kc <= g.iw;
        T.check = (inside && T.K_total % BK == 0) ? 0 : (g.kr * g.kc <= 31 ? 1 : 2);
    } else if (mode == 1) {
        const bool inside = g.kr == 1 && g.kc == 1 && g.pt == 0 && g.pl == 0 && (g.ih - 1) / g.sr < g.oh && (g.iw - 1) / g.sc < g.ow;
        T.check = (inside && T.K_total % BK == 0) ? 0 : (T.rt * T.st_ <= 31 ? 1 : 2);
    }
    // backward-weight of a 1x1, stride-1, unpadded convolution: k = (n, p, q) is contiguous inside an image for x and for dy, so
    // both operands can be gathered with 16-byte loads when groups of four k never straddle an image
    const bool planes_dense = mode == 2 && g.kr == 1 && g.kc == 1 && g.sr == 1 && g.sc == 1 && g.pt == 0 && g.pl == 0 &&
                              g.ih == g.oh && g.iw == g.ow && (g.oh * g.ow) % 4 == 0 && aligned16(srcA) && aligned16(srcB);
    const bool both_rowmajor = planes_dense && T.K_total % BK == 0;
    if (both_rowmajor) T.check = 0;
    // ... and, when the planes are at least one K-block long, both can be copied by TMA straight into the operand ring; the
    // reduction then runs over (image, 32-pixel chunk) and needs neither k nor row tables
    const int w_chunks = (g.oh * g.ow + 31) / 32;
    bool wtma = planes_dense && g_conv_wtma > 0 && g.oh * g.ow >= 32 && g.c >= 32 && g.k >= 32;
    int w_bn = 0;
    if (wtma) {
        w_bn = T.N_total <= 32 ? 32 : (T.N_total <= 64 ? 64 : 128);
        P.chunks_per_image = w_chunks; P.images = g.n; P.raw_hi = g_conv_wtma > 1;
        if (!encode_plane_map(&P.mapA, srcA, g.oh * g.ow, g.c, g.n, BM, true) || !encode_plane_map(&P.mapOut, srcB, g.oh * g.ow, g.k, g.n, w_bn, true)) wtma = false;
    }
    if (wtma) { T.check = 4; T.K_total = 0; T.K_pad = 0; }             // no k tables; check 4 keeps these tables apart in the cache
    int k_pad = wtma ? g.n * w_chunks * BK : T.K_pad;
    // backward-weight of 3x3 stride-1 "same" layers: the dy operand by TMA as above, the x operand built in shared memory from
    // raw slabs that TMA delivers (one per K-block for all nine taps of the tile's 14 channels)
    bool wslab = mode == 2 && g_conv_wslab && g_conv_wtma > 0 && g.kr == 3 && g.kc == 3 && g.sr == 1 && g.sc == 1 && g.pt == 1 && g.pl == 1 &&
                 g.ih == g.oh && g.iw == g.ow && g.iw >= 3 && 2 * (g.iw + 1) + BK + 3 <= WS_SLAB_PX && (g.oh * g.ow) % 4 == 0 && g.oh * g.ow >= 32 &&
                 g.c >= WS_CH && g.k >= 32 && aligned16(srcA) && aligned16(srcB);
    if (wslab) {
        const int ws_bn = T.N_total <= 32 ? 32 : (T.N_total <= 64 ? 64 : 128);
        P.chunks_per_image = w_chunks; P.images = g.n; P.raw_hi = g_conv_wtma > 1; P.img_w = g.iw; P.plane_px = g.oh * g.ow;
        if (!encode_plane_map(&P.mapA, srcA, g.oh * g.ow, g.c, g.n, WS_SLAB_CH, false, WS_SLAB_PX) ||
            !encode_plane_map(&P.mapOut, srcB, g.oh * g.ow, g.k, g.n, ws_bn, true)) wslab = false;
    }
    if (wslab) { T.check = 6; T.K_total = 0; T.K_pad = 0; k_pad = g.n * w_chunks * BK; }      // no k tables; check 6 keeps these tables apart in the cache
    // any backward-weight: dy alone has that property whatever the filter and stride
    const bool b_vector = mode == 2 && (g.oh * g.ow) % 4 == 0 && T.K_total % BK == 0 && aligned16(srcB);
    // forward / backward-data of a 1x1 stride-1 unpadded convolution: rows are pixels of one image plane, k is the channel,
    // so the activation operand and the output are plain [image][channel][pixel] tensors that TMA can move
    const int pq_ = g.oh * g.ow;
    const int a_channels = mode == 0 ? g.c : g.k, o_channels = mode == 0 ? g.k : g.c;
    const int chunks = (pq_ + 31) / 32;
    bool atma = g_conv_tma > 0 && (mode == 0 || mode == 1) && g.kr == 1 && g.kc == 1 && g.sr == 1 && g.sc == 1 && g.pt == 0 && g.pl == 0 &&
                g.ih == g.oh && g.iw == g.ow && pq_ % 4 == 0 && pq_ >= 32 && a_channels >= 32 && o_channels >= 32 &&
                aligned16(srcA) && aligned16(out) && (long long)g.n * chunks * 32 < 0x7fffffffLL &&
                (mode == 0 || out_zero || g_conv_tma > 1);
    if (atma) {
        P.chunks_per_image = chunks; P.images = g.n;
        if (!encode_plane_map(&P.mapA, srcA, pq_, a_channels, g.n) || !encode_plane_map(&P.mapOut, out, pq_, o_channels, g.n)) atma = false;
    }
    if (atma) { T.check = 3; T.M_total = 0; allow_split = false; }      // no row tables; check 3 keeps these tables apart in the cache
    // forward / backward-data of a 3x3 stride-1 "same" convolution: K-blocks ordered (channel group, tap), the nine taps of a group
    // read one raw slab of the plane (tile + halo) that TMA delivers; tiles are 128 consecutive pixels of ONE image
    const int tiles_per_image = (pq_ + BM - 1) / BM;
    bool stma = g_conv_tma > 0 && (mode == 0 || mode == 1) && g.kr == 3 && g.kc == 3 && g.sr == 1 && g.sc == 1 && g.pt == 1 && g.pl == 1 &&
                g.ih == g.oh && g.iw == g.ow && g.iw >= 3 && 2 * g.iw + BM + 5 <= SLAB_PX && pq_ % 4 == 0 && pq_ >= 64 && a_channels >= 32 && o_channels >= 32 &&
                aligned16(srcA) && aligned16(out) && (long long)g.n * tiles_per_image * BM < 0x7fffffffLL && (mode == 0 || out_zero || g_conv_tma > 1) &&
                g_conv_tma3;
    if (stma) {
        P.chunks_per_image = 4 * tiles_per_image; P.images = g.n; P.img_w = g.iw; P.tap_sign = mode == 0 ? 1 : -1;
        if (!encode_plane_map(&P.mapA, srcA, pq_, a_channels, g.n, BK, false, SLAB_PX) || !encode_plane_map(&P.mapOut, out, pq_, o_channels, g.n)) stma = false;
    }
    if (stma) { T.check = 5; T.M_total = 0; allow_split = false; T.K_pad = (a_channels + BK - 1) / BK * 9 * BK; T.K_total = T.K_pad; k_pad = T.K_pad; }
    const int m_rows = atma ? g.n * chunks * 32 : stma ? g.n * tiles_per_image * BM : wslab ? (g.c + WS_CH - 1) / WS_CH * BM : T.M_total;
    // the compact k table keeps 27 bits of offset beside the 5-bit tap number
    if (T.check == 1 && (long long)(g.c > g.k ? g.c : g.k) * (g.ih * g.iw > g.oh * g.ow ? g.ih * g.iw : g.oh * g.ow) + (long long)(g.kr + 1) * (g.iw + g.ow) >= (1ll << 26)) T.check = 2;
    P.check = T.check;
    // 1x1 unpadded layers: the prefetch warp covers pf_rows consecutive rows per touched line (a row step of sc pixels)
    P.pf_rows = 0;
    if (g_conv_prefetch && T.check == 0 && g.kr == 1 && g.kc == 1) {
        if (mode == 1) P.pf_rows = 32;
        else if (mode == 0) P.pf_rows = g.sc == 1 ? 32 : (g.sc == 2 ? 16 : 0);
    }
    const int bn = T.N_total <= 32 ? 32 : (T.N_total <= 64 ? 64 : 128);
    const int tiles_m = (m_rows + BM - 1) / BM, tiles_n = (T.N_total + bn - 1) / bn;
    const int kblocks = k_pad / BK;
    // Split the reduction so that the persistent CTAs finish together: the makespan of `tiles * splits` work items dealt
    // round-robin to the SMs is ceil(items / SMs) rounds of (K-blocks per split + one epilogue); splitting also costs a
    // write and a read of every partial output.  Pick the split count with the smallest estimate (microseconds).
    // The tensor core truncates when it adds into the accumulator, so a chain of accumulations drifts toward zero in
    // proportion to its length (measured on backward-weight of N=64, 256 channels, 56x56: 2000 k-steps per accumulator
    // gave 3e-5 of the largest gradient).  kMaxChainBlocks K-blocks per split keep every accumulator's chain at about
    // 200 k-steps (a few 1e-6); the partial sums of the splits are added in fp32 with rounding.
    constexpr int kMaxChainBlocks = 160;
    const int tiles = tiles_m * tiles_n;
    const int sp_min = allow_split ? (kblocks + kMaxChainBlocks - 1) / kMaxChainBlocks : 1;
    int splits = sp_min;
    if (allow_split && kblocks >= 8) {
        const double t_kblock = mode == 2 ? 2.5 : 1.0, t_epilogue = 3.0;
        int max_splits = kblocks / 4 < 128 ? kblocks / 4 : 128;
        if (max_splits < sp_min) max_splits = sp_min + sp_min / 4;
        double best = 1e30;
        for (int sp = sp_min; sp <= max_splits; sp++) {
            const int kb = (kblocks + sp - 1) / sp;
            const int sp_eff = (kblocks + kb - 1) / kb;
            if (sp_eff != sp) continue;
            const long long rounds = ((long long)tiles * sp + EDDLB200_NUM_SMS - 1) / EDDLB200_NUM_SMS;
            double cost = (double)rounds * (kb * t_kblock + t_epilogue);
            if (sp > 1) cost += 3.0 + 2.0 * (double)out_total * sizeof(float) * sp / 6.0e6;
            if (cost < best * 0.97) { best = cost; splits = sp; }      // prefer fewer splits unless the gain is clear
        }
    }
    const int kbs = (kblocks + splits - 1) / splits;
    splits = (kblocks + kbs - 1) / kbs;
    // one scratch carve-up: tables and split-K partials
    size_t off = 0;
    auto carve = [&](size_t bytes) { size_t o = off; off += (bytes + 255) & ~size_t(255); return o; };
    const size_t o_rowA = carve((size_t)T.M_total * 8), o_kA = carve((size_t)T.K_pad * 8), o_rowB = carve((size_t)T.N_total * 4),
                 o_kB = carve((size_t)T.K_pad * 4), o_kC = carve((size_t)T.K_pad * 4), o_outM = carve((size_t)T.M_total * 4);
    const size_t table_bytes = off;
    // cached tables live in their own allocation; the scratch arena then holds only partials and packed weights
    char *tb = nullptr; bool build = true;
    {
        TableCache &tc = g_tables[dev];
        std::lock_guard<std::mutex> lock(tc.mu);
        const auto key = table_key(T);
        auto it = tc.entries.find(key);
        if (it != tc.entries.end()) { tb = it->second; build = false; }
        else if (tc.bytes + table_bytes <= kTableCacheBudget && cudaMalloc((void **)&tb, table_bytes) == cudaSuccess) {
            tc.entries.emplace(key, tb); tc.bytes += table_bytes;
        } else { tb = nullptr; cudaGetLastError(); }
    }
    if (tb) off = 0;
    const bool tb_cached = tb != nullptr;
    const size_t o_part = carve(splits > 1 ? out_total * splits * sizeof(float) : 0),
                 o_pack = carve(mode != 2 ? (size_t)kblocks * tiles_n * bn * BK * sizeof(float) * (precision != 1 ? 2 : 1) : 0);
    char *ws = (char *)scratch(cx, off ? off : 256);
    if (!ws) return cudaErrorMemoryAllocation;
    if (!tb) tb = ws;
    if (!g_status[dev]) {
        if (cudaMalloc((void **)&g_status[dev], sizeof(int)) != cudaSuccess) return cudaErrorMemoryAllocation;
        cudaMemsetAsync(g_status[dev], 0, sizeof(int), st);
    }
    T.rowA = (int2 *)(tb + o_rowA); T.kA = (int2 *)(tb + o_kA); T.rowB = (int *)(tb + o_rowB); T.kB = (int *)(tb + o_kB); T.outM = (int *)(tb + o_outM); T.kC = (int *)(tb + o_kC);
    if (build) {
        const long long entries = (long long)T.M_total + T.K_pad + T.N_total;
        build_tables_kernel<<<grid_for((size_t)entries, 256), 256, 0, st>>>(T);
        EB_LAUNCH_CHECK("conv_tc(tables)");
    }
    P.packedB = nullptr;
    // which coordinate of B is contiguous in memory (the pack kernel reads along it): the in-channel row for backward-data,
    // n for a GEMM whose B is not transposed
    const bool b_row_fastest = mode == 1 || (mode == 4 && !g.iw);
    if (mode != 2) {
        const float *img = tb_cached ? packed_weights(cx, st, dev, table_key(T), bn, precision, srcB, (size_t)g.k * g.c * g.kr * g.kc * sizeof(float),
                                                       T.rowB, T.kB, kblocks, tiles_n, T.N_total, b_row_fastest) : nullptr;
        if (!img) {
            // no cached image (tables not cached, cache full, or allocation failed): pack into the scratch arena for this call
            dim3 pgrid(kblocks, tiles_n);
            pack_b_kernel<<<pgrid, 256, 0, st>>>(srcB, T.rowB, T.kB, (float *)(ws + o_pack), bn, T.N_total, tiles_n, b_row_fastest, precision);
            EB_LAUNCH_CHECK("conv_tc(pack weights)");
            img = (const float *)(ws + o_pack);
        }
        P.packedB = img;
    }
    P.srcA = srcA; P.srcB = srcB;
    P.rowA = T.rowA; P.kA = T.kA; P.rowB = T.rowB; P.kB = T.kB; P.outM = T.outM; P.kC = T.kC;
    P.M_total = wslab ? T.M_total : m_rows; P.N_total = T.N_total; P.K_pad = k_pad;      // slab-fed backward-weight: the real (channel, tap) count
    P.kblocks_per_split = kbs;
    P.tiles_m = tiles_m; P.tiles_n = tiles_n; P.splits = splits;
    // a single accumulator drifts by ~2.5e-6 at 64 k-steps (K = 512); longer chains rotate over three
    P.nmain = (kbs * (BK / 8) > 64) ? NMAIN : 1;
    P.status = g_status[dev];
    if (splits > 1) { P.out = (float *)(ws + o_part); P.split_stride = (long long)out_total; P.accumulate = 0; P.bias = nullptr; }
    else { P.out = out; P.split_stride = 0; P.accumulate = mode == 4 ? T.ca == 1 : ((mode == 1 || mode == 2) && !out_zero); P.add_zero = out_zero; P.bias = bias; }
    P.reduce_out = (atma || stma) && P.accumulate;
    const long long total_tiles = (long long)tiles_m * tiles_n * splits;
    dim3 grid((unsigned)(total_tiles < EDDLB200_NUM_SMS ? total_tiles : EDDLB200_NUM_SMS), 1, 1);
    int r;
    // backward-weight has no bf16 variant: precision 2 runs it as precision 0
    if (wtma) r = precision != 1 ? launch_bn<0, false, true, 2>(cx, st, P, grid, bn, dev) : launch_bn<1, false, true, 2>(cx, st, P, grid, bn, dev);
    else if (wslab) r = precision != 1 ? launch_bn<0, false, true, 4>(cx, st, P, grid, bn, dev) : launch_bn<1, false, true, 4>(cx, st, P, grid, bn, dev);
    else if (mode == 2 && both_rowmajor) r = precision != 1 ? launch_bn<0, false, true>(cx, st, P, grid, bn, dev) : launch_bn<1, false, true>(cx, st, P, grid, bn, dev);
    else if (mode == 2 && b_vector) r = precision != 1 ? launch_bn<0, true, true>(cx, st, P, grid, bn, dev) : launch_bn<1, true, true>(cx, st, P, grid, bn, dev);
    else if (mode == 2) r = precision != 1 ? launch_bn<0, true>(cx, st, P, grid, bn, dev) : launch_bn<1, true>(cx, st, P, grid, bn, dev);
    else if (stma) r = precision == 0 ? launch_bn<0, false, false, 3>(cx, st, P, grid, bn, dev)
                   : precision == 2 ? launch_bn<2, false, false, 3>(cx, st, P, grid, bn, dev) : launch_bn<1, false, false, 3>(cx, st, P, grid, bn, dev);
    else if (atma) r = precision == 0 ? launch_bn<0, false, false, 1>(cx, st, P, grid, bn, dev)
                   : precision == 2 ? launch_bn<2, false, false, 1>(cx, st, P, grid, bn, dev) : launch_bn<1, false, false, 1>(cx, st, P, grid, bn, dev);
    else if (precision == 0) r = launch_bn<0, false>(cx, st, P, grid, bn, dev);
    else if (precision == 2) r = launch_bn<2, false>(cx, st, P, grid, bn, dev);
    else r = launch_bn<1, false>(cx, st, P, grid, bn, dev);
    if (r) return r;
    if (splits > 1) {
        if (mode == 0 || out_zero || (mode == 4 && T.ca != 1)) {
            // `out` holds nothing to add to: store the sum of the partials (0 + p0 + p1 + ...)
            splitk_store_kernel<<<grid_for(out_total, 256), 256, 0, st>>>((const float *)(ws + o_part), out, out_total, splits, mode == 0 ? bias : nullptr, g.oh * g.ow, g.k);
            EB_LAUNCH_CHECK("conv_tc(split-K store)");
            return 0;
        }
        return splitk_reduce_accumulate(cx, st, (const float *)(ws + o_part), out, out_total, splits);
    }
    return 0;
}

int run(DevCtx *cx, cudaStream_t st, int dev, int mode, const ConvGeom &g, const float *srcA, const float *srcB, float *out,
        const float *bias, int precision, bool out_zero = false) {
    const int pq = g.oh * g.ow, hw = g.ih * g.iw, rs = g.kr * g.kc;
    TableArgs T{};
    T.g = g; T.mode = mode;
    TcParams P{};
    if (mode == 0) {
        T.M_total = g.n * pq; T.N_total = g.k; T.K_total = g.c * rs; P.limY = g.ih; P.limX = g.iw; P.out_n_stride = pq;
        return run_one(cx, st, dev, T, P, srcA, srcB, out, bias, precision, (size_t)g.n * g.k * pq, true);
    }
    if (mode == 2) {
        T.M_total = g.c * rs; T.N_total = g.k; T.K_total = g.n * pq; P.limY = g.ih; P.limX = g.iw; P.out_n_stride = g.c * rs;
        return run_one(cx, st, dev, T, P, srcA, srcB, out, nullptr, precision, (size_t)g.k * g.c * rs, true, out_zero);
    }
    // backward-data: one dense problem per residue class of the strides
    P.limY = g.oh; P.limX = g.ow; P.out_n_stride = hw; T.N_total = g.c;
    for (int ca = 0; ca < g.sr; ca++)
        for (int cb = 0; cb < g.sc; cb++) {
            T.ca = ca; T.cb = cb;
            T.y0 = ((ca - g.pt) % g.sr + g.sr) % g.sr; T.x0 = ((cb - g.pl) % g.sc + g.sc) % g.sc;
            T.hc = T.y0 < g.ih ? (g.ih - T.y0 + g.sr - 1) / g.sr : 0;
            T.wc = T.x0 < g.iw ? (g.iw - T.x0 + g.sc - 1) / g.sc : 0;
            T.rt = ca < g.kr ? (g.kr - ca + g.sr - 1) / g.sr : 0;
            T.st_ = cb < g.kc ? (g.kc - cb + g.sc - 1) / g.sc : 0;
            T.M_total = g.n * T.hc * T.wc; T.K_total = g.k * T.rt * T.st_;
            if (T.M_total == 0 || T.K_total == 0) continue;       // this class receives nothing
            const bool dense = (g.sr == 1 && g.sc == 1);
            if (int r = run_one(cx, st, dev, T, P, srcA, srcB, out, nullptr, precision, (size_t)g.n * g.c * hw, dense, dense && out_zero)) return r;
        }
    return 0;
}

// Gather-form col2im for the GEMM route of backward-data: dx[n,c,y,x] += sum over the taps (r,s) of the pixel's stride
// residue class of T[n][(c,r,s)][p][q], p = (y+pt-r)/sr, q = (x+pl-s)/sc.  One thread per dx element, no atomics.
__global__ void __launch_bounds__(256) col2im_gather_kernel(ConvGeom g, const float *__restrict__ T, float *__restrict__ dx) {
    const int hw = g.ih * g.iw, pq = g.oh * g.ow, rs = g.kr * g.kc;
    const long long total = (long long)g.n * g.c * hw;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int x = (int)(i % g.iw);
        long long t = i / g.iw;
        const int y = (int)(t % g.ih); t /= g.ih;          // t = n*C + c
        const int r0 = (y + g.pt) % g.sr, s0 = (x + g.pl) % g.sc;
        const int p0 = (y + g.pt - r0) / g.sr, q0 = (x + g.pl - s0) / g.sc;
        const float *plane = T + (size_t)t * rs * pq;
        float acc = 0.f;
        for (int r = r0, p = p0; r < g.kr && p >= 0; r += g.sr, p--) {
            if (p >= g.oh) continue;
            for (int s = s0, q = q0; s < g.kc && q >= 0; s += g.sc, q--) {
                if (q >= g.ow) continue;
                acc += __ldg(plane + (size_t)(r * g.kc + s) * pq + p * g.ow + q);
            }
        }
        dx[i] = __fadd_rn(dx[i], acc);
    }
}

// out[c][r] = in[r][c] for a small rows x cols matrix (the weight tensor of a few-channel layer)
__global__ void __launch_bounds__(256) transpose_kernel(const float *__restrict__ in, float *__restrict__ out, int rows, int cols) {
    const size_t total = (size_t)rows * cols, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int c = (int)(i / rows), r = (int)(i - (size_t)c * rows);
        out[i] = __ldg(in + (size_t)r * cols + c);
    }
}

// Backward-data for layers with very few input channels (the 7x7 stem: C = 3).  With pixels on M and channels on N the
// GEMM would gather every dy value for 3 useful columns out of 32; instead T[(n,p,q)][(c,r,s)] = sum_f dy * w is one dense
// GEMM that reads dy exactly once (K = filters), followed by the gather-form col2im above.
int run_small_c_bwd_data(DevCtx *cx, cudaStream_t st, int dev, const ConvGeom &g, const float *dy, const float *w, float *dx, int precision) {
    const int pq = g.oh * g.ow, rs = g.kr * g.kc;
    const size_t t_elems = (size_t)g.n * g.c * rs * pq;
    // T lives in a buffer of its own: run_one() re-carves the scratch arena
    static float *tbuf[EDDLB200_MAX_DEVICES] = {}; static size_t tcap[EDDLB200_MAX_DEVICES] = {};
    if (tcap[dev] < t_elems) {
        cudaStreamSynchronize(st);
        if (tbuf[dev]) cudaFree(tbuf[dev]);
        tbuf[dev] = nullptr; tcap[dev] = 0;
        if (cudaMalloc((void **)&tbuf[dev], t_elems * sizeof(float)) != cudaSuccess) { cudaGetLastError(); return 1; }
        tcap[dev] = t_elems;
    }
    // The GEMM is a 1x1 stride-1 convolution of dy ([image][filter][pixel], the filters as input channels) with the weights
    // transposed to [(c, r, s)][filter]: with a transposed copy of the (small) weight tensor it runs on the TMA-fed kernel,
    // whose epilogue hands whole blocks to TMA stores -- this GEMM has two K-blocks per tile and writes 12 times what it reads
    static float *wt[EDDLB200_MAX_DEVICES] = {}; static size_t wcap[EDDLB200_MAX_DEVICES] = {};
    const size_t w_elems = (size_t)g.k * g.c * rs;
    bool dense = g_conv_tma > 0 && pq % 4 == 0 && pq >= 32 && g.k >= 32 && g.c * rs >= 32 && pq < 16000 * 16000;
    if (dense && wcap[dev] < w_elems) {
        cudaStreamSynchronize(st);
        if (wt[dev]) cudaFree(wt[dev]);
        wt[dev] = nullptr; wcap[dev] = 0;
        if (cudaMalloc((void **)&wt[dev], w_elems * sizeof(float)) != cudaSuccess) { cudaGetLastError(); dense = false; }
        else wcap[dev] = w_elems;
    }
    if (dense) {
        transpose_kernel<<<grid_for(w_elems, 256), 256, 0, st>>>(w, wt[dev], g.k, g.c * rs);
        EB_LAUNCH_CHECK("conv_tc(transpose weights)");
        if (watch_any(cx)) note_write(cx, wt[dev], w_elems * sizeof(float));       // the packed image of the copy is stale now
        // the plane as one row of pq pixels: a 1x1 layer does not care about its two-dimensional shape
        const ConvGeom g1{g.n, g.k, 1, pq, g.c * rs, 1, 1, 1, pq, 1, 1, 0, 0};
        const int r = pq < 16000 ? run(cx, st, dev, 0, g1, dy, wt[dev], tbuf[dev], nullptr, precision) : 1;
        if (r != 0 && r != 1) return r;
        dense = r == 0;
    }
    if (!dense) {
        TableArgs T{};
        T.g = g; T.mode = 3;
        TcParams P{};
        T.M_total = g.n * pq; T.N_total = g.c * rs; T.K_total = g.k; P.limY = 1; P.limX = 1; P.out_n_stride = pq;
        if (int r = run_one(cx, st, dev, T, P, dy, w, tbuf[dev], nullptr, precision, t_elems, false)) return r;
    }
    col2im_gather_kernel<<<grid_for((size_t)g.n * g.c * g.ih * g.iw, 256), 256, 0, st>>>(g, tbuf[dev], dx);
    EB_LAUNCH_CHECK("conv_tc(col2im gather)");
    return 0;
}

bool fits(const ConvGeom &g) {
    // index tables hold 16-bit coordinates and 32-bit offsets
    return g.ih < 16000 && g.iw < 16000 && g.oh < 16000 && g.ow < 16000;
}

}  // namespace

namespace eb {

int conv_tc_fwd(DevCtx *cx, cudaStream_t st, const ConvGeom &g, const float *x, const float *w, const float *bias, float *y, int precision) {
    if (!fits(g)) return 1;
    int dev = 0; cudaGetDevice(&dev);
    return run(cx, st, dev, 0, g, x, w, y, bias, precision);
}

int conv_tc_bwd_data(DevCtx *cx, cudaStream_t st, const ConvGeom &g, const float *dy, const float *w, float *dx, int precision, bool dx_zero) {
    if (!fits(g)) return 1;
    int dev = 0; cudaGetDevice(&dev);
    const bool small_c = g.c <= 8 && (size_t)g.n * g.c * g.kr * g.kc * g.oh * g.ow < (size_t(1) << 29);
    if (dx_zero && (small_c || g.sr != 1 || g.sc != 1)) {
        // these routes add into dx piecewise: write the zeros the caller still owes it
        if (int r = launch_zero_fill(cx, st, dx, (size_t)g.n * g.c * g.ih * g.iw)) return r;
        dx_zero = false;
    }
    if (g.c <= 8 && (size_t)g.n * g.c * g.kr * g.kc * g.oh * g.ow < (size_t(1) << 29)) {
        const int r = run_small_c_bwd_data(cx, st, dev, g, dy, w, dx, precision);
        if (r != 1) return r;
    }
    return run(cx, st, dev, 1, g, dy, w, dx, nullptr, precision, dx_zero);
}

int conv_tc_bwd_weight(DevCtx *cx, cudaStream_t st, const ConvGeom &g, const float *x, const float *dy, float *gw, int precision, bool gw_zero) {
    if (!fits(g)) return 1;
    int dev = 0; cudaGetDevice(&dev);
    return run(cx, st, dev, 2, g, x, dy, gw, nullptr, precision, gw_zero);
}

// C[m x n] (row-major) = op(A) op(B), += when inc_c == 1, written into known zeros when inc_c == 2: the dense layers' GEMMs
// (Tensor::mult2D, src/tensor/tensor_math.cpp) on the same kernel, as a "convolution" whose rows are the rows of op(A).
// 1 = not taken (the caller falls back to the fp32 FMA GEMM).
int conv_tc_gemm(DevCtx *cx, cudaStream_t st, const float *a, int ta, const float *b, int tb, float *c, int inc_c, int m, int n, int k, int precision) {
    if ((long long)m * k >= 0x7fffffffLL || (long long)n * k >= 0x7fffffffLL || (long long)m * n >= 0x7fffffffLL) return 1;
    int dev = 0; cudaGetDevice(&dev);
    TableArgs T{};
    T.g = ConvGeom{m, k, ta ? 1 : 0, tb ? 1 : 0, n, 1, 1, 1, 1, 1, 1, 0, 0};
    T.mode = 4; T.ca = inc_c;
    TcParams P{};
    T.M_total = m; T.N_total = n; T.K_total = k; P.limY = 1; P.limX = 1; P.out_n_stride = 1;
    return run_one(cx, st, dev, T, P, a, b, c, nullptr, precision, (size_t)m * n, true, inc_c == 2);
}

int conv_tc_set_prefetch(int on) { g_conv_prefetch = on ? 1 : 0; return 0; }
int conv_tc_set_tma(int level) { g_conv_tma = level < 0 ? 0 : (level > 2 ? 2 : level); return 0; }
int conv_tc_set_pack_cache(int on) { g_conv_pack_cache = on ? 1 : 0; return 0; }
int conv_tc_set_tma_3x3(int on) { g_conv_tma3 = on ? 1 : 0; return 0; }
int conv_tc_set_tma_wgrad_3x3(int on) { g_conv_wslab = on ? 1 : 0; return 0; }
int conv_tc_set_tma_wgrad(int level) { g_conv_wtma = level < 0 ? 0 : (level > 2 ? 2 : level); return 0; }

// 0 = no kernel of this file has timed out on the device since the last call
int conv_tc_status(int dev, cudaStream_t st, int *out) {
    *out = 0;
    if (!g_status[dev]) return 0;
    cudaError_t e = cudaMemcpyAsync(out, g_status[dev], sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e == cudaSuccess && *out) e = cudaMemsetAsync(g_status[dev], 0, sizeof(int), st);
    return e == cudaSuccess ? 0 : (int)e;
}

}  // namespace eb

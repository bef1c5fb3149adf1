// The one contraction kernel of this library: a persistent, warp-specialised
// implicit-GEMM for sm_100a.  One CTA per SM (or one cluster of two) walks a static list of output tiles.
//
//   warps 0, 6  TMA producers  : tiled cp.async.bulk.tensor loads (never multicast) into a ring of
//                                128-byte-swizzled shared-memory stages; warp 0 fetches the A
//                                operand, warp 6 the B operand (issuing a TMA costs its thread a
//                                few hundred clocks, so one thread cannot feed narrow tiles)
//   warp 1      MMA issuer     : one thread issues tcgen05.mma, accumulators live in TMEM,
//                                two TMEM buffers so the epilogue of tile i overlaps tile i+1
//   warps 2..5  epilogue       : tcgen05.ld -> bias / rounding / cast -> TMA or plain global stores
//   warps 7..10 epilogue       : second group, TMA-store instances only, used on short-K tiles
//
// Two tile walks share the pipeline:
//   MODE_FPROP  rows of the tile are output pixels (n, h, w) taken as one TMA box of the
//               NHWC activation; the K loop runs over (tap, channel block) with stride,
//               padding and dilation folded into the box coordinates (out-of-range reads are
//               zero-filled by TMA).  Covers Conv2d forward, Conv2d input-gradient and
//               ConvTranspose2d forward (one sub-problem per output phase, no col2im),
//               ConvTranspose2d input-gradient, and plain GEMMs (Linear forward / dgrad)
//               seen as a 1x1 convolution over an image of height 1.  Unit-stride walks with
//               several taps use the patch walk instead (see KParams::patch).
//   MODE_WGRAD  rows of the tile are (tap, patch channel), columns are the other tensor's
//               channels, the K loop runs over pixels; both operands are MN-major boxes of the
//               NHWC tensors.  Each split-K slice stores its partial sums into its own plane of a
//               scratch buffer; a second kernel adds the planes in slice order (no atomics).
//               Covers Conv2d / ConvTranspose2d weight-gradient and Linear weight-gradient.
// 256-wide tiles of long-K problems run as CTA pairs (cta_group::2, see the kernel's comment).
#pragma once
#include "nml_ptx.cuh"

namespace nml {

enum { MODE_FPROP = 0, MODE_WGRAD = 1 };
enum { OUT_NHWC = 0, OUT_NCHW = 1, OUT_NHWC_TMA = 2, OUT_NCHW_TMA = 3 };  // _TMA: written by TMA stores
#define NML_IS_TMA_OUT(m) ((m) == OUT_NHWC_TMA || (m) == OUT_NCHW_TMA)
enum { KIND_F16 = 0, KIND_TF32 = 2 };

// Error codes written to the status word by a kernel that gave up on a wait.
enum {
    ERR_WAIT_EMPTY = 101,
    ERR_WAIT_FULL = 102,
    ERR_WAIT_TMEM_EMPTY = 103,
    ERR_WAIT_TMEM_FULL = 104,
    ERR_WAIT_DRAIN = 105
};

constexpr int kMaxPhases = 16;
constexpr int kMaxTaps = 128;
constexpr int kTileM = 128;
constexpr int kStageABytes = kTileM * 128;
constexpr int kThreads = 224;      // warp 0: A loads, warp 1: MMA issue, warps 2-5: epilogue, warp 6: B loads
constexpr int kThreadsWide = 352;  // TMA-store instances: warps 7-10 are a second epilogue group (used when the
                                   // K loop is short and the epilogue is the critical path; they need few registers)
__host__ __device__ constexpr int threads_for(int out_mode) { return (out_mode == 2 || out_mode == 3) ? kThreadsWide : kThreads; }
constexpr int kStagingBufBytes = 4096;         // one staging buffer: 32 rows x 128 bytes of output
constexpr int kBiasTileBytes = 8 * 256 * 4;   // per epilogue warp (up to 8): the current tile's bias values

struct Tap {
    short dh, dw;  // offset of this tap's box from the tile origin, in input pixels
    int wk;        // first K index (fprop) / tap index (wgrad) of this tap in the weight operand
    int aoff;      // patch walk: where this tap's rows start inside the patch, in 16-byte units
};

struct Phase {
    short ph, pw;        // first output row / column of the phase
    short tap_begin, tap_count;
    short org_h, org_w;  // patch walk: smallest tap offset of the phase (its patch origin relative to the tile origin)
    int hq, wq;          // extent of the phase grid
    int tiles_h, tiles_w;
    int tile_begin;      // first tile id of this phase
    unsigned long long mul_w, mul_h;  // 2^40 / tiles_w + 1, 2^40 / tiles_h + 1 (division by multiplication)
};

struct KParams {
    CUtensorMap tmA[2];  // fprop: activation (plane 0 = value or tf32 "hi", plane 1 = tf32 "lo")
                         // wgrad: the tensor patches are cut from
    CUtensorMap tmB[2];  // fprop: weights; wgrad: the plainly indexed tensor
    CUtensorMap tmC;     // OUT_NHWC_TMA: the output, box = the 32 rows x 128 bytes one epilogue warp owns
    int mode, out_mode;
    int num_tiles, n_tiles;
    unsigned long long mul_nt;  // 2^40 / n_tiles + 1
    int fastdiv;         // 1: tile ids and divisors are small enough for the multiply-and-shift division to be exact
    int bn;              // UMMA N of one tile
    int stages;
    int cm_bw_log2, cm_bh_log2;  // OUT_NCHW_TMA: pixel sub-box (w, h) of one epilogue warp's 32 rows
    int epi_warps;       // 4, or 8 on the TMA-store instances when the epilogue is the critical path
    int pair;            // 1: launched as clusters of two CTAs sharing 256x256 tiles (cta_group::2)
    int stg_bufs;        // staging buffers per epilogue warp (4 KB each): 2 when shared memory allows, else 1
    int ka;              // K atoms (128-byte-wide operand slices) per stage; narrow tiles take 2 to amortise the
                         // per-stage barrier round trip over 8 MMAs
    int a_mn_major, b_mn_major;
    int a_grouped, b_grouped;  // MN-major operand fetched as ONE box whose outermost dimension walks
                               // the 128-byte column groups (needs the channel count to be a multiple of kb)
    // Patch walk (forward walk, unit stride, several taps): instead of one 128-row box per tap, the A
    // producer loads ONE box per channel block that covers the tile's 8 x 16 output pixels plus the reach
    // of every tap, and the MMA of tap (dh, dw) reads its 128 rows straight out of that patch: its
    // descriptor starts (dh * patch_w + dw) rows in, and 8-row groups are patch_w rows apart.  (The swizzle
    // is a function of the shared-memory address, so a descriptor may start on any 128-byte row.)
    // A is then read from L2 about once instead of once per tap.  B slices stream through the stage ring,
    // or stay resident in shared memory for the whole launch when all of them fit.
    // Forward walk, few tiles and a long K loop (U-Net bottleneck layers): the K iterations of a tile are
    // cut into fsplit slices that run as separate tiles; slice z stores its partial sums into plane z
    // of a row-major scratch, and a small pass adds the planes in order and produces the output.
    int fsplit;          // K slices per tile (1 = off)
    int base_tiles;      // tiles of one slice; tile id = slice * base_tiles + tile
    // Phase-packed gather walk (strided input gradients / transposed forwards with very few output
    // channels): the stride_h x stride_w output phases are packed into the tile's columns, column
    // j = (ph * shuf_sw + pw) * shuf_c + c, so the walk is ONE unit-stride pass over the input whose row
    // (n, i, j) scatters to out[n][shuf_sh*i + ph][shuf_sw*j + pw][c] (row-major output only).
    int shuf_sh, shuf_sw;  // 0 = off
    int shuf_c, shuf_oh, shuf_ow;
    // Weight-gradient patch walk (unit column stride, one 64-channel group per tap): a CTA owns a slice of
    // the K blocks (8 x 8 pixels of one image) and ALL row tiles of the gradient at once.  Per K block it
    // loads one haloed patch of the tensor the taps are cut from and one box of the other tensor; row tile
    // i = taps (2i, 2i+1) is an MN-major descriptor into the patch (start = the first tap's rows, the second
    // tap's 64 columns LBO = their row distance away, 8-pixel groups one patch row * stride_h apart) and
    // accumulates into its own TMEM columns [i * bn, (i+1) * bn).  Each tensor is then read from L2 about
    // once instead of once per tap / once per row tile.
    int wpatch;          // 1: weight-gradient patch walk
    int w_mtiles;        // row tiles (accumulators), w_mtiles * bn <= 512
    int w_coalesce;      // 1: the partial gradient leaves through shared memory as contiguous runs of stores
                         //    (needs 32 gradient columns, 32 * c_patch * taps floats, to fit in the operand ring)
    int patch;           // 1: patch walk
    int patch_w, patch_h;    // patch extent in pixels
    int patch_bytes;     // bytes one patch buffer occupies (multiple of 1024)
    int a_stages;        // patch buffers
    int b_resident;      // 1: every B slice of the launch is loaded once, at [pass plane][cb][tap] * bn * 128
    int issuers;         // resident patch walk: 2 = the B producer issues the odd tiles (needs a_stages >= 2 * c_blocks)
    int ring_bytes;      // bytes of the operand ring(s) in front of the staging buffers
    int a_ring_off;      // patch walk: offset of the patch buffers within the ring region
    int kind;            // KIND_F16 / KIND_TF32
    int passes;          // 1, or 3 for the 3xTF32 split (hi*lo, lo*hi, hi*hi in that order)
    int kb;              // elements per 128-byte row (64 fp16, 32 tf32)
    int c_blocks;        // channel blocks of kb per tap (fprop) / per patch tensor (wgrad)
    int wb_log2, hb_log2, nb_log2;  // fprop: M-tile box; wgrad: K-block pixel box
    int batch;
    int a_stride_h, a_stride_w;      // multiplier of the tile origin in A coordinates (conv stride)
    int out_stride_h, out_stride_w;  // distance between neighbouring outputs of one phase
    int n_phases;
    // wgrad
    int groups_total;    // taps * c_blocks column groups of kb patch channels
    int split_k, kblocks_total, ktiles_h, ktiles_w;
    int c_patch, c_plain, n_taps;
    int kw_pack;         // wgrad, few-channel path: patch index j of a tap means (kw = j / 8, c = j % 8)
    int kw_count;        //   ... with kw_count valid kw per tap row; dW index = ((plain*C + c)*KH + kh)*KW + kw
    int m_fastest;       // wgrad tile order: consecutive CTAs share the plain operand's columns (re-read the smaller tensor)
    // epilogue
    void* out;
    const float* bias;
    int bias_f16;        // 1: `bias` points at fp16 values (TMA-store epilogues only)
    int out_f16, round_f16;
    int c_out;           // valid columns
    int out_h, out_w;    // output image
    int ld_out;          // NHWC: elements between consecutive pixels
    int* err;
    unsigned long long wait_limit_ns;  // time limit of one bounded wait; 0 = the built-in default
    // Partial sums of K slices (split-K weight gradient, K-split forward walk) are never added with
    // atomics: slice z stores its partial tile into plane z of `out` (planes are plane_elems floats
    // apart) and a second kernel adds the planes in slice order, so results are bitwise repeatable.
    // wgrad planes are laid out [plain channel][ld_plane rows of the tile walk] (patch walk: like dW).
    unsigned long long plane_elems;
    int ld_plane;
    Phase phases[kMaxPhases];
    Tap taps[kMaxTaps];
};

// Tile decode runs once per tile in every role, and the epilogue warps in particular are bound by
// instruction issue: a runtime integer division is ~25 instructions, the multiply-and-shift 4.
// Exact for x * d < 2^40 (the host checks).
__device__ __forceinline__ uint32_t fast_div(uint32_t x, unsigned long long mul) {
    return static_cast<uint32_t>((static_cast<unsigned long long>(x) * mul) >> 40);
}
// Forward walk: tile index within its phase -> column tile and the (w, h, n) position of the row tile.
template <bool kPair>
__device__ __forceinline__ void decode_fprop_tile(const KParams& P, const Phase& ph, int local, uint32_t cta_rank,
                                                  int& ntile, int& tw, int& th, int& tn) {
    uint32_t m = P.fastdiv ? fast_div(local, P.mul_nt) : static_cast<uint32_t>(local) / P.n_tiles;
    ntile = local - static_cast<int>(m) * P.n_tiles;
    if (kPair) m = 2 * m + cta_rank;  // the pair's two row tiles
    const uint32_t q = P.fastdiv ? fast_div(m, ph.mul_w) : m / ph.tiles_w;
    tw = static_cast<int>(m - q * ph.tiles_w);
    const uint32_t n = P.fastdiv ? fast_div(q, ph.mul_h) : q / ph.tiles_h;
    th = static_cast<int>(q - n * ph.tiles_h);
    tn = static_cast<int>(n);
}

// Tile id -> (column tile, row tile, K slice) of a weight-gradient launch.
__device__ __forceinline__ void decode_wgrad_tile(const KParams& P, int tile, int m_tiles, int& ntile, int& mt, int& z) {
    const int mn = m_tiles * P.n_tiles;
    z = tile / mn;
    const int r = tile - z * mn;
    if (P.m_fastest) {
        ntile = r / m_tiles;
        mt = r - ntile * m_tiles;
    } else {
        mt = r / P.n_tiles;
        ntile = r - mt * P.n_tiles;
    }
}

__device__ __forceinline__ float round_through_f16(float v) {
    return __half2float(__float2half_rn(v));
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr)
                 : "memory");
    return v;
}
__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Stores 32 (or fewer) consecutive output columns of one accumulator row.
__device__ __noinline__ void store_row_chunk(const KParams& P, const float (&v)[32], size_t row_off,
                                                size_t col_stride, int cg, int ncols) {
    if (P.out_mode == OUT_NHWC) {
        if (P.out_f16) {
            __half* o = reinterpret_cast<__half*>(P.out) + row_off + cg;
            if (ncols == 32 && (P.ld_out & 7) == 0) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint4 pk;
                    __half2 h0 = __floats2half2_rn(v[8 * q + 0], v[8 * q + 1]);
                    __half2 h1 = __floats2half2_rn(v[8 * q + 2], v[8 * q + 3]);
                    __half2 h2 = __floats2half2_rn(v[8 * q + 4], v[8 * q + 5]);
                    __half2 h3 = __floats2half2_rn(v[8 * q + 6], v[8 * q + 7]);
                    pk.x = *reinterpret_cast<uint32_t*>(&h0);
                    pk.y = *reinterpret_cast<uint32_t*>(&h1);
                    pk.z = *reinterpret_cast<uint32_t*>(&h2);
                    pk.w = *reinterpret_cast<uint32_t*>(&h3);
                    reinterpret_cast<uint4*>(o)[q] = pk;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (j < ncols) o[j] = __float2half_rn(v[j]);
            }
        } else {
            float* o = reinterpret_cast<float*>(P.out) + row_off + cg;
            if (ncols == 32 && (P.ld_out & 3) == 0) {
#pragma unroll
                for (int q = 0; q < 8; ++q)
                    reinterpret_cast<float4*>(o)[q] =
                        make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (j < ncols) o[j] = v[j];
            }
        }
    } else {  // OUT_NCHW: lanes are consecutive pixels, so each column store coalesces
        if (P.out_f16) {
            __half* o = reinterpret_cast<__half*>(P.out) + row_off + static_cast<size_t>(cg) * col_stride;
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < ncols) o[j * col_stride] = __float2half_rn(v[j]);
        } else {
            float* o = reinterpret_cast<float*>(P.out) + row_off + static_cast<size_t>(cg) * col_stride;
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < ncols) o[j * col_stride] = v[j];
        }
    }
}

// Specialised on the tile walk, the output layout and the output type so that each instance's hot
// loops stay small: the epilogue warps run alone on their schedulers and stall on instruction fetch
// when the straight-line code of every variant is laid out in one kernel.
// kPair: two CTAs of a cluster compute one 256-row x 256-column tile with cta_group::2 MMAs issued by
// the rank-0 CTA; each CTA loads its own 128 rows of A and its own 128-column half of B (no multicast),
// which halves the B traffic and the MMA issue cost per SM and leaves room for 6 stages.
template <int kMode, int kOutMode, bool kOutF16, bool kPair>
__global__ void __launch_bounds__(threads_for(kOutMode), 1) umma_conv_kernel(const __grid_constant__ KParams P) {
    extern __shared__ uint8_t smem_raw[];
    // stages need 1024-byte alignment for the 128-byte swizzle pattern
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    const uint32_t cta_rank = kPair ? cluster_ctarank() : 0u;
    const bool leader = (cta_rank == 0);
    const int tile_first = kPair ? (blockIdx.x >> 1) : blockIdx.x;
    const int tile_step = kPair ? (gridDim.x >> 1) : gridDim.x;
    const int stage_b_bytes = (kPair ? P.bn / 2 : P.bn) * 128;   // one atom of B (a pair member holds half the columns)
    const int stage_bytes = P.ka * (kStageABytes + stage_b_bytes);  // [A atoms][B atoms]
    const int b_off = P.ka * kStageABytes;                        // first B atom within a stage
    uint8_t* staging = smem + P.ring_bytes;  // epilogue warps x 4 KB
    const int staging_bytes = P.epi_warps * P.stg_bufs * kStagingBufBytes;
    float* bias_tile = reinterpret_cast<float*>(staging + staging_bytes);
    uint8_t* ctrl = staging + staging_bytes + kBiasTileBytes;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctrl);          // [stages]
    uint64_t* empty_bar = full_bar + 8;                               // [stages]
    uint64_t* tfull_bar = empty_bar + 8;                              // [2]
    uint64_t* tempty_bar = tfull_bar + 2;                             // [2]
    uint64_t* afull_bar = tempty_bar + 2;                             // [4] patch walk: patch buffers
    uint64_t* aempty_bar = afull_bar + 4;                             // [4]
    uint64_t* bres_bar = aempty_bar + 4;                              // [1] patch walk: resident B has landed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bres_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 2);  // abort state: 4 ints, 8-byte aligned

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // two accumulators; the epilogue reads 32 columns at a time, so a 16-column tile still needs 16 + 32
    const uint32_t tmem_need = P.wpatch ? P.w_mtiles * P.bn : (P.bn < 32) ? P.bn + 32 : 2 * P.bn;
    const uint32_t tmem_cols = (tmem_need <= 32) ? 32 : (tmem_need <= 64) ? 64 : (tmem_need <= 128) ? 128
                               : (tmem_need <= 256) ? 256 : 512;

    if (threadIdx.x == 0) {
        for (int s = 0; s < P.stages; ++s) {
            mbar_init(smem_u32(&full_bar[s]), P.patch ? 1 : 2);  // one arrival (with its byte count) per producer warp
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&tfull_bar[b]), 1);
            mbar_init(smem_u32(&tempty_bar[b]), (kPair ? 2 : 1) * P.epi_warps);  // the leader also hears the partner's epilogue warps
        }
        for (int s = 0; s < 4; ++s) {
            mbar_init(smem_u32(&afull_bar[s]), P.wpatch ? 4 : 1);  // weight-gradient patch walk: the four epilogue warps meet here
            mbar_init(smem_u32(&aempty_bar[s]), 1);
        }
        mbar_init(smem_u32(bres_bar), 1);
        abort_state_init(abort_flag, P.wait_limit_ns);
        fence_mbar_init();
        tma_prefetch_desc(&P.tmA[0]);
        tma_prefetch_desc(&P.tmB[0]);
        if (P.passes > 1) {
            tma_prefetch_desc(&P.tmA[1]);
            tma_prefetch_desc(&P.tmB[1]);
        }
    }
    if (warp == 1) {
        if (kPair) {
            tmem_alloc_pair(smem_u32(tmem_slot), tmem_cols);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(smem_u32(tmem_slot), tmem_cols);
            tmem_relinquish();
        }
    }
    tc_fence_before();
    __syncthreads();
    if (kPair) cluster_sync_all();  // the partner's barriers must be initialised before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int box_bytes = P.kb * 128;  // one MN-major box: kb k-rows of 128 bytes
    const int wb = 1 << P.wb_log2, hb = 1 << P.hb_log2;

    // Patch walk with resident B: the MMA issue loop of the tiles t_first, t_first + t_step, ... of this CTA.
    // Nothing in it waits for B, so two warps can share the issuing: the MMA warp takes the even tiles
    // (accumulator 0) and the B producer, idle once the weights have landed, the odd ones (accumulator 1).
    // One warp's per-tile bookkeeping (barrier waits, commits) then hides behind the other's MMAs.
    // A parity wait is only meaningful if the barrier's previous phase is known to be over.  An issuer waits
    // for a patch only after the epilogue has drained tile t - 2 (the accumulator it reuses), i.e. after every
    // patch up to that tile's last has landed; with a_stages >= 2 * c_blocks the patch that used the same
    // buffer before is among those (or is this issuer's own), so the host allows two issuers only then.
    auto patch_resident_issue = [&](int t_first, int t_step) {
        const uint32_t idesc = make_instr_desc(P.kind, 0, P.b_mn_major, kTileM, P.bn);
        const bool b32 = P.b_mn_major && P.kind == KIND_TF32;
        const uint32_t lbo_b = P.b_mn_major ? box_bytes : 16;
        const uint32_t adv_b = P.b_mn_major ? (((P.kind == KIND_F16) ? 16 : 8) * 128) >> 4 : 2;
        const uint32_t b_step = static_cast<uint32_t>(stage_b_bytes) >> 4;
        const uint32_t sbo_a = static_cast<uint32_t>(P.patch_w * P.a_stride_h) * 128u;  // 8-row groups: one output row = a_stride_h patch rows apart
        const bool f16 = (P.kind == KIND_F16);
        if (!mbar_wait(smem_u32(bres_bar), 0, abort_flag, P.err, ERR_WAIT_FULL)) return;
        int titer = t_first;
        int p = 0;
        for (int tile = tile_first + t_first * tile_step; tile < P.num_tiles; tile += t_step * tile_step, titer += t_step) {
            while (p + 1 < P.n_phases && tile >= P.phases[p + 1].tile_begin) ++p;
            const Tap* tp = &P.taps[P.phases[p].tap_begin];
            const int nt = P.phases[p].tap_count;
            const int tb0 = P.phases[p].tap_begin;
            const int buf = titer & 1;
            const uint32_t tpar = (titer >> 1) & 1;
            if (!mbar_wait(smem_u32(&tempty_bar[buf]), tpar ^ 1, abort_flag, P.err, ERR_WAIT_TMEM_EMPTY)) return;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + buf * P.bn;
            uint32_t acc = 0;
            for (int cb = 0; cb < P.c_blocks; ++cb) {
                const int pi = titer * P.c_blocks + cb;  // patches are consumed in tile order
                const int pstage = pi % P.a_stages;
                const uint32_t pparity = (pi / P.a_stages) & 1;
                if (!mbar_wait(smem_u32(&afull_bar[pstage]), pparity, abort_flag, P.err, ERR_WAIT_FULL)) return;
                tc_fence_after();
                if (elect_one()) {
                    const uint64_t adesc0 = make_smem_desc(smem_u32(smem + P.a_ring_off) + pstage * P.patch_bytes, 16, sbo_a, 2);
                    uint64_t bdesc = make_smem_desc(smem_u32(smem) + (cb * P.n_taps + tb0) * stage_b_bytes, lbo_b, b32 ? 512 : 1024, b32 ? 1 : 2);
#pragma unroll 1
                    for (int t = 0; t < nt; ++t) {
                        const uint64_t adesc = adesc0 + static_cast<uint32_t>(tp[t].aoff);
                        if (f16) {
                            umma_f16(d_tmem, adesc, bdesc, idesc, acc);
                            umma_f16(d_tmem, adesc + 2, bdesc + adv_b, idesc, 1u);
                            umma_f16(d_tmem, adesc + 4, bdesc + 2 * adv_b, idesc, 1u);
                            umma_f16(d_tmem, adesc + 6, bdesc + 3 * adv_b, idesc, 1u);
                        } else {
                            umma_tf32(d_tmem, adesc, bdesc, idesc, acc);
                            umma_tf32(d_tmem, adesc + 2, bdesc + adv_b, idesc, 1u);
                            umma_tf32(d_tmem, adesc + 4, bdesc + 2 * adv_b, idesc, 1u);
                            umma_tf32(d_tmem, adesc + 6, bdesc + 3 * adv_b, idesc, 1u);
                        }
                        acc = 1u;
                        bdesc += b_step;
                    }
                    umma_commit(smem_u32(&aempty_bar[pstage]));
                    if (cb + 1 == P.c_blocks) {
                        umma_commit(smem_u32(&tfull_bar[buf]));
                    }
                }
                acc = 1u;
                __syncwarp();
            }
        }
    };

    // ------------------------------------------------------------ producer --
    if (warp == 0 || warp == 6) {
        const bool do_a = (warp == 0), do_b = (warp == 6);
        // Issuing one TMA keeps its thread busy for ~300 clocks, more than the MMAs of a narrow K atom last.
        // The atoms of a stage are therefore issued by one lane each, in the same instruction (the patch
        // walk, with one box per tile, is driven by lane 0 alone).
        // Weight-gradient operands that cannot be fetched as one box per K block get a lane per box.
        const int boxes_per_atom = (kMode != MODE_WGRAD || kPair) ? 1
                                   : do_a ? (P.a_grouped ? 1 : kTileM / P.kb) : (P.b_grouped ? 1 : P.bn / P.kb);
        const int issue_lanes = (P.patch || P.wpatch) ? 1 : P.ka * boxes_per_atom;
        const uint32_t issue_mask = (1u << issue_lanes) - 1u;
        if (kMode == MODE_FPROP && !kPair && P.patch && P.b_resident && do_b) {
            // Resident weights: every slice once, for the whole launch (one column tile, one pass plane, K-major
            // repacked weights).  The slices are spread over the lanes of the warp, so the dozens of TMA issues at
            // the start of the kernel cost one thread's worth of them, not their sum.
            const uint32_t fb = smem_u32(bres_bar);
            const int slices = P.c_blocks * P.n_taps;
            if (lane == 0) mbar_arrive_expect_tx(fb, static_cast<uint32_t>(slices) * stage_b_bytes);
            __syncwarp();
            for (int i = lane; i < slices; i += 32) {
                const int cb = i / P.n_taps, t = i - cb * P.n_taps;  // slot order [cb][tap of every phase]
                tma_load_2d(smem_u32(smem) + i * stage_b_bytes, &P.tmB[0], fb, P.taps[t].wk + cb * P.kb, 0);
            }
            __syncwarp();
        }
        if (lane < issue_lanes) {
            int stage = 0;
            uint32_t parity = 0;
            bool ok = true;
            int issued = 0;
            const uint32_t a_bytes = kStageABytes;
            const uint32_t tx_bytes = do_a ? a_bytes : stage_b_bytes;  // this producer's share of one atom
            // B slice of (tap, channel block, column tile) -> shared memory at sb
            auto load_b = [&](uint32_t sb, const CUtensorMap* tb, uint32_t fb, const Tap& tap, int cb, int ntile) {
                if (!P.b_mn_major) {
                    tma_load_2d(sb, tb, fb, tap.wk + cb * P.kb, ntile * P.bn);
                } else if (P.b_grouped) {
                    tma_load_3d(sb, tb, fb, 0, tap.wk + cb * P.kb, (ntile * P.bn) / P.kb);
                } else {
                    int nb = P.bn / P.kb;
                    for (int j = 0; j < nb; ++j)
                        tma_load_2d(sb + j * box_bytes, tb, fb, ntile * P.bn + j * P.kb, tap.wk + cb * P.kb);
                }
            };
            if (kMode == MODE_FPROP && !kPair && P.patch) {  // (issue_lanes == 1 here)
                if (do_a) {
                    const uint32_t a_base = smem_u32(smem + P.a_ring_off);
                    const uint32_t patch_tx = static_cast<uint32_t>(P.patch_w) * P.patch_h * 128u;
                    int abuf = 0;
                    uint32_t apar = 0;
                    int p = 0;
                    for (int tile = tile_first; ok && tile < P.num_tiles; tile += tile_step) {
                        while (p + 1 < P.n_phases && tile >= P.phases[p + 1].tile_begin) ++p;
                        const Phase& pt = P.phases[p];
                        int nt_unused, tw, th, tn;
                        decode_fprop_tile<false>(P, pt, tile - pt.tile_begin, 0u, nt_unused, tw, th, tn);
                        const int w0 = (tw << P.wb_log2) * P.a_stride_w + pt.org_w;
                        const int h0 = (th << P.hb_log2) * P.a_stride_h + pt.org_h;
                        for (int pass = 0; ok && pass < P.passes; ++pass) {
                            const CUtensorMap* ta = &P.tmA[(P.passes == 3 && pass == 1) ? 1 : 0];
                            for (int cb = 0; cb < P.c_blocks; ++cb) {
                                if (!mbar_wait(smem_u32(&aempty_bar[abuf]), apar ^ 1, abort_flag, P.err, ERR_WAIT_EMPTY)) {
                                    ok = false;
                                    break;
                                }
                                const uint32_t fb = smem_u32(&afull_bar[abuf]);
                                mbar_arrive_expect_tx(fb, patch_tx);
                                tma_load_4d(a_base + abuf * P.patch_bytes, ta, fb, cb * P.kb, w0, h0, tn);
                                ++issued;
                                if (++abuf == P.a_stages) {
                                    abuf = 0;
                                    apar ^= 1;
                                }
                            }
                        }
                    }
                    if (!ok) {  // give patches already requested a bounded chance to land
                        int back = issued < P.a_stages ? issued : P.a_stages;
                        for (int i = 0; i < back; ++i) {
                            if (--abuf < 0) {
                                abuf = P.a_stages - 1;
                                apar ^= 1;
                            }
                            uint64_t t0 = globaltimer_ns();
                            while (!mbar_try_wait(smem_u32(&afull_bar[abuf]), apar)) {
                                if (globaltimer_ns() - t0 > 2000000ull) {
                                    atomicCAS(P.err, 0, ERR_WAIT_DRAIN);
                                    break;
                                }
                            }
                        }
                    }
                    ok = true;   // nothing left for the common unwinding below
                    issued = 0;
                } else if (P.b_resident) {
                    // (the slices were requested above, by the whole warp)
                    const uint32_t fb = smem_u32(bres_bar);
                    // the MMA warp waits for these before its first tile; if it gave up, wait here (bounded) so
                    // that no copy is in flight when the CTA's shared memory goes away
                    uint64_t t0 = globaltimer_ns();
                    while (!mbar_try_wait(fb, 0)) {
                        if (globaltimer_ns() - t0 > 4000000ull) {
                            if (*abort_flag) atomicCAS(P.err, 0, ERR_WAIT_DRAIN);
                            break;
                        }
                    }
                } else {
                    // B streams through the ring, P.ka tap slices per stage
                    int p = 0;
                    for (int tile = tile_first; ok && tile < P.num_tiles; tile += tile_step) {
                        while (p + 1 < P.n_phases && tile >= P.phases[p + 1].tile_begin) ++p;
                        const Phase& pt = P.phases[p];
                        const int ntile = (tile - pt.tile_begin) % P.n_tiles;
                        for (int pass = 0; ok && pass < P.passes; ++pass) {
                            const CUtensorMap* tb = &P.tmB[(P.passes == 3 && pass == 0) ? 1 : 0];
                            for (int cb = 0; ok && cb < P.c_blocks; ++cb)
                                for (int t = 0; t < pt.tap_count; t += P.ka) {
                                    if (!mbar_wait(smem_u32(&empty_bar[stage]), parity ^ 1, abort_flag, P.err, ERR_WAIT_EMPTY)) {
                                        ok = false;
                                        break;
                                    }
                                    const int n = min(P.ka, pt.tap_count - t);
                                    const uint32_t fb = smem_u32(&full_bar[stage]);
                                    mbar_arrive_expect_tx(fb, n * stage_b_bytes);
                                    for (int j = 0; j < n; ++j)
                                        load_b(smem_u32(smem) + (stage * P.ka + j) * stage_b_bytes, tb, fb,
                                               P.taps[pt.tap_begin + t + j], cb, ntile);
                                    ++issued;
                                    if (++stage == P.stages) {
                                        stage = 0;
                                        parity ^= 1;
                                    }
                                }
                        }
                    }
                }
            } else
            for (int tile_id = tile_first; ok && tile_id < P.num_tiles; tile_id += tile_step) {
                int tile = tile_id, kz = 0;
                if (kMode == MODE_FPROP && P.fsplit > 1) {
                    kz = tile_id / P.base_tiles;
                    tile = tile_id - kz * P.base_tiles;
                }
                if (kMode == MODE_FPROP) {
                    int p = 0;
                    while (p + 1 < P.n_phases && tile >= P.phases[p + 1].tile_begin) ++p;
                    const Phase& ph = P.phases[p];
                    int local = tile - ph.tile_begin;
                    int ntile, tw, th, tn;
                    decode_fprop_tile<kPair>(P, ph, local, cta_rank, ntile, tw, th, tn);
                    int w0 = (tw << P.wb_log2) * P.a_stride_w;
                    int h0 = (th << P.hb_log2) * P.a_stride_h;
                    int n0 = tn << P.nb_log2;
                    int k_iters = P.passes * ph.tap_count * P.c_blocks;
                    int k_first = 0;
                    if (P.fsplit > 1) {  // this slice's share of the K iterations
                        const int per = (k_iters + P.fsplit - 1) / P.fsplit;
                        k_first = min(kz * per, k_iters);
                        k_iters = min(k_first + per, k_iters) - k_first;
                    }
                    // this lane's position in the K loop, (pass, tap, channel block) of iteration it + lane, kept
                    // by counting: a division per stage is time the 256-wide tiles' producer does not have
                    int pass = 0, t = 0, cb = 0;
                    auto advance = [&](int steps) {
                        cb += steps;
                        while (cb >= P.c_blocks) {
                            cb -= P.c_blocks;
                            if (++t == ph.tap_count) {
                                t = 0;
                                ++pass;
                            }
                        }
                    };
                    advance(k_first + lane);
                    for (int it = 0; it < k_iters; it += P.ka) {  // one stage per iteration
                        // in a pair every load signals the LEADER's barrier, which expects both members' bytes
                        uint32_t fb = smem_u32(&full_bar[stage]);
                        if (kPair) fb = map_to_cta(fb, 0);
                        // (the issuing lanes leave together: a lane must never wait in __syncwarp for one that gave up)
                        if (!__all_sync(issue_mask, mbar_wait(smem_u32(&empty_bar[stage]), parity ^ 1, abort_flag, P.err,
                                                              ERR_WAIT_EMPTY))) {
                            ok = false;
                            break;
                        }
                        const int n_in_stage = min(P.ka, k_iters - it);
                        if (lane == 0) {
                            if (!kPair) mbar_arrive_expect_tx(fb, n_in_stage * tx_bytes);
                            else if (leader) mbar_arrive_expect_tx(smem_u32(&full_bar[stage]), 2 * n_in_stage * tx_bytes);
                        }
                        __syncwarp(issue_mask);
                        if (lane < n_in_stage) {  // this lane's atom: K iteration it + lane = (pass, tap, channel block)
                            const Tap& tap = P.taps[ph.tap_begin + t];
                            // 3xTF32 order: hi*lo, lo*hi, then hi*hi -- the small cross terms go in
                            // while the accumulator is small, so the tensor core's truncating
                            // accumulation costs them nothing
                            const CUtensorMap* ta = &P.tmA[(P.passes == 3 && pass == 1) ? 1 : 0];
                            const CUtensorMap* tb = &P.tmB[(P.passes == 3 && pass == 0) ? 1 : 0];
                            const uint32_t sa = smem_u32(smem + stage * stage_bytes) + lane * kStageABytes;
                            const uint32_t sb = smem_u32(smem + stage * stage_bytes) + b_off + lane * stage_b_bytes;
                            if (kPair) {
                                const int ncol = ntile * P.bn + static_cast<int>(cta_rank) * (P.bn / 2);  // this member's half of B
                                if (do_a) tma_load_4d_pair(sa, ta, fb, cb * P.kb, w0 + tap.dw, h0 + tap.dh, n0);
                                if (do_b) {
                                    if (!P.b_mn_major) tma_load_2d_pair(sb, tb, fb, tap.wk + cb * P.kb, ncol);
                                    else tma_load_3d_pair(sb, tb, fb, 0, tap.wk + cb * P.kb, ncol / P.kb);
                                }
                            } else if (do_a) {
                                tma_load_4d(sa, ta, fb, cb * P.kb, w0 + tap.dw, h0 + tap.dh, n0);
                            } else {
                                load_b(sb, tb, fb, tap, cb, ntile);
                            }
                        }
                        advance(P.ka);
                        ++issued;
                        if (++stage == P.stages) {
                            stage = 0;
                            parity ^= 1;
                        }
                    }
                } else if (!kPair && P.wpatch) {  // MODE_WGRAD, patch walk: stage = [patch][box of the other tensor]
                    const int ntile = tile % P.n_tiles, z = tile / P.n_tiles;
                    const int per = (P.kblocks_total + P.split_k - 1) / P.split_k;
                    const int kb_begin = z * per, kb_end = min(kb_begin + per, P.kblocks_total);
                    int tw = kb_begin % P.ktiles_w;
                    int th = (kb_begin / P.ktiles_w) % P.ktiles_h;
                    int tn = kb_begin / (P.ktiles_w * P.ktiles_h);
                    const uint32_t w_stage = static_cast<uint32_t>(P.patch_bytes) + stage_b_bytes;
                    const uint32_t patch_tx = static_cast<uint32_t>(P.patch_w) * P.patch_h * 128u;
                    for (int kbi = kb_begin; kbi < kb_end; ++kbi) {
                        if (!mbar_wait(smem_u32(&empty_bar[stage]), parity ^ 1, abort_flag, P.err, ERR_WAIT_EMPTY)) {
                            ok = false;
                            break;
                        }
                        const uint32_t fb = smem_u32(&full_bar[stage]);
                        const int w0 = tw << 3, h0 = th << 3;
                        const uint32_t st_addr = smem_u32(smem) + stage * w_stage;
                        if (do_a) {
                            mbar_arrive_expect_tx(fb, patch_tx);
                            tma_load_4d(st_addr, &P.tmA[0], fb, 0, w0 * P.a_stride_w + P.phases[0].org_w,
                                        h0 * P.a_stride_h + P.phases[0].org_h, tn);
                        } else {
                            mbar_arrive_expect_tx(fb, stage_b_bytes);
                            tma_load_5d(st_addr + P.patch_bytes, &P.tmB[0], fb, 0, w0, h0, tn, (ntile * P.bn) / P.kb);
                        }
                        ++issued;
                        if (++stage == P.stages) {
                            stage = 0;
                            parity ^= 1;
                        }
                        if (++tw == P.ktiles_w) {
                            tw = 0;
                            if (++th == P.ktiles_h) {
                                th = 0;
                                ++tn;
                            }
                        }
                    }
                } else {  // MODE_WGRAD
                    int m_tiles = (P.groups_total * P.kb + kTileM - 1) / kTileM;
                if (kPair) m_tiles = (m_tiles + 1) / 2;  // tile ids name pairs of row tiles
                    int ntile, mt, z;
                    decode_wgrad_tile(P, tile, m_tiles, ntile, mt, z);
                    if (kPair) mt = 2 * mt + static_cast<int>(cta_rank);
                    int per = (P.kblocks_total + P.split_k - 1) / P.split_k;
                    int kb_begin = z * per;
                    int kb_end = min(kb_begin + per, P.kblocks_total);
                    int g_per_tile = kTileM / P.kb;
                    int na = g_per_tile, nb = P.bn / P.kb;
                    if (kPair) {
                    // one K block and one box per stage: the single issuing lane has ~500 clocks per
                    // stage, so its loop carries nothing but counters
                    int left = P.passes * max(kb_end - kb_begin, 0);  // K iterations still to load for this tile
                    int slot = 0, n_in_stage = 0;
                    for (int pass = 0; ok && pass < P.passes; ++pass) {
                        const CUtensorMap* ta = &P.tmA[(P.passes == 3 && pass == 1) ? 1 : 0];
                        const CUtensorMap* tb = &P.tmB[(P.passes == 3 && pass == 0) ? 1 : 0];
                        int tw = kb_begin % P.ktiles_w;
                        int th = (kb_begin / P.ktiles_w) % P.ktiles_h;
                        int tn = kb_begin / (P.ktiles_w * P.ktiles_h);
                        // groups of this M tile: with a_grouped they share one tap
                        const int g0 = min(mt * g_per_tile, P.groups_total - 1);
                        const int t0 = g0 / P.c_blocks;
                        const int cib0 = g0 - t0 * P.c_blocks;
                        for (int kbi = kb_begin; kbi < kb_end; ++kbi) {
                            int w0 = tw << P.wb_log2, h0 = th << P.hb_log2, n0 = tn << P.nb_log2;
                            uint32_t fb = smem_u32(&full_bar[stage]);
                            if (kPair) fb = map_to_cta(fb, 0);
                            if (slot == 0) {
                                if (!mbar_wait(smem_u32(&empty_bar[stage]), parity ^ 1, abort_flag,
                                               P.err, ERR_WAIT_EMPTY)) {
                                    ok = false;
                                    break;
                                }
                                n_in_stage = min(P.ka, left);
                                if (!kPair) mbar_arrive_expect_tx(fb, n_in_stage * tx_bytes);
                                else if (leader) mbar_arrive_expect_tx(smem_u32(&full_bar[stage]), 2 * n_in_stage * tx_bytes);
                            }
                            --left;
                            uint32_t sa = smem_u32(smem + stage * stage_bytes) + slot * kStageABytes;
                            uint32_t sb = smem_u32(smem + stage * stage_bytes) + b_off + slot * stage_b_bytes;
                            if (kPair) {  // pairs are only planned for grouped operands
                                const Tap& tap = P.taps[t0];
                                if (do_a)
                                    tma_load_5d_pair(sa, ta, fb, 0, w0 * P.a_stride_w + tap.dw, h0 * P.a_stride_h + tap.dh, n0,
                                                     cib0);
                                if (do_b)
                                    tma_load_5d_pair(sb, tb, fb, 0, w0, h0, n0,
                                                     (ntile * P.bn) / P.kb + static_cast<int>(cta_rank) * (P.bn / 2 / P.kb));
                            } else
                            if (!do_a) {
                            } else if (P.a_grouped) {
                                const Tap& tap = P.taps[t0];
                                tma_load_5d(sa, ta, fb, 0, w0 * P.a_stride_w + tap.dw, h0 * P.a_stride_h + tap.dh, n0,
                                            cib0);
                            } else {
                                for (int g = 0; g < na; ++g) {
                                    int gi = min(mt * g_per_tile + g, P.groups_total - 1);
                                    int t = gi / P.c_blocks;
                                    int cib = gi - t * P.c_blocks;
                                    const Tap& tap = P.taps[t];
                                    tma_load_4d(sa + g * box_bytes, ta, fb, cib * P.kb,
                                                w0 * P.a_stride_w + tap.dw, h0 * P.a_stride_h + tap.dh, n0);
                                }
                            }
                            if (kPair || !do_b) {
                            } else if (P.b_grouped) {
                                tma_load_5d(sb, tb, fb, 0, w0, h0, n0, (ntile * P.bn) / P.kb);
                            } else {
                                for (int j = 0; j < nb; ++j)
                                    tma_load_4d(sb + j * box_bytes, tb, fb, ntile * P.bn + j * P.kb, w0,
                                                h0, n0);
                            }
                            if (++slot == n_in_stage) {
                                slot = 0;
                                ++issued;
                                if (++stage == P.stages) {
                                    stage = 0;
                                    parity ^= 1;
                                }
                            }
                            if (++tw == P.ktiles_w) {
                                tw = 0;
                                if (++th == P.ktiles_h) {
                                    th = 0;
                                    ++tn;
                                }
                            }
                        }
                    }
                    } else {
                    const int nkb = max(kb_end - kb_begin, 0);
                    const int k_total = P.passes * nkb;  // K iterations of this tile: (pass, K block)
                    // groups of this M tile: with a_grouped they share one tap
                    const int g0 = min(mt * g_per_tile, P.groups_total - 1);
                    const int t0 = g0 / P.c_blocks;
                    const int cib0 = g0 - t0 * P.c_blocks;
                    // this lane's K iteration (it + lane) as (pass, K block -> pixel box), kept by counting
                    const int tw0 = kb_begin % P.ktiles_w;
                    const int th0 = (kb_begin / P.ktiles_w) % P.ktiles_h;
                    const int tn0 = kb_begin / (P.ktiles_w * P.ktiles_h);
                    int pass = 0, rel = 0, tw = tw0, th = th0, tn = tn0;
                    auto advance = [&](int steps) {
                        for (int i = 0; i < steps; ++i) {
                            if (++rel >= nkb) {
                                rel = 0;
                                ++pass;
                                tw = tw0;
                                th = th0;
                                tn = tn0;
                            } else if (++tw == P.ktiles_w) {
                                tw = 0;
                                if (++th == P.ktiles_h) {
                                    th = 0;
                                    ++tn;
                                }
                            }
                        }
                    };
                    const int my_atom = lane / boxes_per_atom, my_box = lane - my_atom * boxes_per_atom;
                    if (nkb > 0) advance(my_atom);
                    for (int it = 0; it < k_total; it += P.ka) {  // one stage per iteration
                        uint32_t fb = smem_u32(&full_bar[stage]);
                        if (kPair) fb = map_to_cta(fb, 0);
                        if (!__all_sync(issue_mask, mbar_wait(smem_u32(&empty_bar[stage]), parity ^ 1, abort_flag, P.err,
                                                              ERR_WAIT_EMPTY))) {
                            ok = false;
                            break;
                        }
                        const int n_in_stage = min(P.ka, k_total - it);
                        if (lane == 0) {
                            if (!kPair) mbar_arrive_expect_tx(fb, n_in_stage * tx_bytes);
                            else if (leader) mbar_arrive_expect_tx(smem_u32(&full_bar[stage]), 2 * n_in_stage * tx_bytes);
                        }
                        __syncwarp(issue_mask);
                        if (my_atom < n_in_stage) {
                            const CUtensorMap* ta = &P.tmA[(P.passes == 3 && pass == 1) ? 1 : 0];
                            const CUtensorMap* tb = &P.tmB[(P.passes == 3 && pass == 0) ? 1 : 0];
                            const int w0 = tw << P.wb_log2, h0 = th << P.hb_log2, n0 = tn << P.nb_log2;
                            const uint32_t sa = smem_u32(smem + stage * stage_bytes) + my_atom * kStageABytes;
                            const uint32_t sb = smem_u32(smem + stage * stage_bytes) + b_off + my_atom * stage_b_bytes;
                            if (kPair) {  // pairs are only planned for grouped operands
                                const Tap& tap = P.taps[t0];
                                if (do_a)
                                    tma_load_5d_pair(sa, ta, fb, 0, w0 * P.a_stride_w + tap.dw, h0 * P.a_stride_h + tap.dh, n0,
                                                     cib0);
                                if (do_b)
                                    tma_load_5d_pair(sb, tb, fb, 0, w0, h0, n0,
                                                     (ntile * P.bn) / P.kb + static_cast<int>(cta_rank) * (P.bn / 2 / P.kb));
                            } else if (do_a) {
                                if (P.a_grouped) {
                                    const Tap& tap = P.taps[t0];
                                    tma_load_5d(sa, ta, fb, 0, w0 * P.a_stride_w + tap.dw, h0 * P.a_stride_h + tap.dh, n0,
                                                cib0);
                                } else {  // this lane's 64-channel group of the row tile
                                    const int g = my_box;
                                    int gi = min(mt * g_per_tile + g, P.groups_total - 1);
                                    int t = gi / P.c_blocks;
                                    int cib = gi - t * P.c_blocks;
                                    const Tap& tap = P.taps[t];
                                    tma_load_4d(sa + g * box_bytes, ta, fb, cib * P.kb,
                                                w0 * P.a_stride_w + tap.dw, h0 * P.a_stride_h + tap.dh, n0);
                                }
                            } else if (P.b_grouped) {
                                tma_load_5d(sb, tb, fb, 0, w0, h0, n0, (ntile * P.bn) / P.kb);
                            } else {  // this lane's 64-column group of the column tile
                                tma_load_4d(sb + my_box * box_bytes, tb, fb, ntile * P.bn + my_box * P.kb, w0, h0, n0);
                            }
                        }
                        advance(P.ka);
                        ++issued;
                        if (++stage == P.stages) {
                            stage = 0;
                            parity ^= 1;
                        }
                    }
                    }
                }
            }
            if (!ok && lane == 0) {
                // Unwinding: give copies already issued a bounded chance to land before the
                // CTA's shared memory goes away.
                int back = issued < P.stages ? issued : P.stages;
                int s = stage;
                uint32_t par = parity;
                for (int i = 0; i < back; ++i) {
                    if (--s < 0) {
                        s = P.stages - 1;
                        par ^= 1;
                    }
                    uint64_t t0 = globaltimer_ns();
                    while (!mbar_try_wait(smem_u32(&full_bar[s]), par)) {
                        if (globaltimer_ns() - t0 > 2000000ull) {
                            atomicCAS(P.err, 0, ERR_WAIT_DRAIN);
                            break;
                        }
                    }
                }
            }
        }
        if (kMode == MODE_FPROP && !kPair && P.patch && P.b_resident && P.issuers == 2 && warp == 6) {
            __syncwarp();
            patch_resident_issue(1, 2);  // the weights are in: help with the odd tiles
        }
    }
    // ---------------------------------------------------------- MMA issuer --
    else if (warp == 1) {
        // The whole warp walks the loop (so loop state and descriptors stay warp-uniform and every
        // lane observes the barriers itself); one elected lane issues the MMAs and their commits.  The loop
        // body is kept minimal: one MMA must be issued every 128 clocks to keep the tensor pipe
        // busy, and everything here is on that single thread's critical path.
        const uint32_t idesc = make_instr_desc(P.kind, P.a_mn_major, P.b_mn_major, kPair ? 2 * kTileM : kTileM, P.bn);
        const uint32_t lbo_a = P.a_mn_major ? box_bytes : 16;
        const uint32_t lbo_b = P.b_mn_major ? box_bytes : 16;
        const int umma_k = (P.kind == KIND_F16) ? 16 : 8;
        // MN-major tf32 operands use the 32-byte-chunk flavour of the 128-byte swizzle
        const bool a32 = P.a_mn_major && P.kind == KIND_TF32;
        const bool b32 = P.b_mn_major && P.kind == KIND_TF32;
        // descriptor start-address advance per UMMA, in 16-byte units
        const uint32_t adv_a = P.a_mn_major ? (umma_k * 128) >> 4 : 2;
        const uint32_t adv_b = P.b_mn_major ? (umma_k * 128) >> 4 : 2;
        const uint64_t adesc0 = make_smem_desc(smem_u32(smem), lbo_a, a32 ? 512 : 1024, a32 ? 1 : 2);
        const uint64_t bdesc0 = make_smem_desc(smem_u32(smem) + b_off, lbo_b, b32 ? 512 : 1024, b32 ? 1 : 2);
        const uint32_t a_atom_step = static_cast<uint32_t>(kStageABytes) >> 4;
        const uint32_t b_atom_step = static_cast<uint32_t>(stage_b_bytes) >> 4;
        const uint32_t stage_step = static_cast<uint32_t>(stage_bytes) >> 4;
        const bool f16 = (P.kind == KIND_F16);
        int stage = 0, pstage = 0;
        uint32_t parity = 0, pparity = 0;
        bool ok = true;
        int titer = 0;
        if (kMode == MODE_FPROP && !kPair && P.patch && P.b_resident) {
            patch_resident_issue(0, P.issuers);
        } else
        for (int tile_id = tile_first; ok && (!kPair || leader) && tile_id < P.num_tiles; tile_id += tile_step, ++titer) {
            int tile = tile_id, kz = 0;
            if (kMode == MODE_FPROP && P.fsplit > 1) {
                kz = tile_id / P.base_tiles;
                tile = tile_id - kz * P.base_tiles;
            }
            int k_iters;
            if (kMode == MODE_FPROP) {
                int p = 0;
                while (p + 1 < P.n_phases && tile >= P.phases[p + 1].tile_begin) ++p;
                k_iters = P.passes * P.phases[p].tap_count * P.c_blocks;
                if (P.fsplit > 1) {
                    const int per = (k_iters + P.fsplit - 1) / P.fsplit;
                    const int k_first = min(kz * per, k_iters);
                    k_iters = min(k_first + per, k_iters) - k_first;
                }
            } else {
                int m_tiles = (P.groups_total * P.kb + kTileM - 1) / kTileM;
                if (kPair) m_tiles = (m_tiles + 1) / 2;  // tile ids name pairs of row tiles
                int z = tile / (P.n_tiles * m_tiles);
                int per = (P.kblocks_total + P.split_k - 1) / P.split_k;
                int kb_begin = z * per;
                int kb_end = min(kb_begin + per, P.kblocks_total);
                k_iters = P.passes * max(kb_end - kb_begin, 0);
            }
            const int buf = titer & 1;
            const uint32_t tpar = (titer >> 1) & 1;
            if (kMode == MODE_WGRAD && !kPair && P.wpatch) {
                // all row tiles at once, accumulator i in columns [i * bn, (i + 1) * bn); no second TMEM buffer, so
                // the epilogue of the previous tile (if this CTA has one) must be over
                const int z = tile / P.n_tiles;
                const int per = (P.kblocks_total + P.split_k - 1) / P.split_k;
                const int nkb = max(min(z * per + per, P.kblocks_total) - z * per, 0);
                if (!mbar_wait(smem_u32(&tempty_bar[0]), (titer & 1) ^ 1, abort_flag, P.err, ERR_WAIT_TMEM_EMPTY)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t w_stage = static_cast<uint32_t>(P.patch_bytes) + stage_b_bytes;
                const uint32_t sbo_a = static_cast<uint32_t>(P.patch_w * P.a_stride_h) * 128u;  // next pixel row of the K block
                // Row tile i = taps (2i, 2i+1): its descriptor relative to stage 0, built once (a 64-column MMA
                // lasts 48 clocks: the K loop has no time to build descriptors).
                uint64_t ad[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int t0 = min(2 * i, P.groups_total - 1), t1 = min(2 * i + 1, P.groups_total - 1);
                    const uint32_t a0 = static_cast<uint32_t>(P.taps[t0].aoff), a1 = static_cast<uint32_t>(P.taps[t1].aoff);
                    ad[i] = make_smem_desc(smem_u32(smem) + (a0 << 4), (a1 - a0) << 4, sbo_a, 2);
                }
                const uint64_t bd0 = make_smem_desc(smem_u32(smem) + P.patch_bytes, box_bytes, 1024, 2);
                const uint32_t a_step = (2u * sbo_a) >> 4;  // two pixel rows = 16 pixels = one MMA's K
                const uint32_t stage_step16 = w_stage >> 4;
                uint32_t accw = 0;
                for (int kbi = 0; kbi < nkb; ++kbi) {
                    if (!mbar_wait(smem_u32(&full_bar[stage]), parity, abort_flag, P.err, ERR_WAIT_FULL)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    if (elect_one()) {
                        const uint64_t so = static_cast<uint64_t>(stage * stage_step16);
                        const uint64_t bdesc = bd0 + so;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            if (i < P.w_mtiles) {
                                const uint64_t adesc = ad[i] + so;
                                const uint32_t d = tmem_base + i * P.bn;
                                umma_f16(d, adesc, bdesc, idesc, accw);
                                umma_f16(d, adesc + a_step, bdesc + adv_b, idesc, 1u);
                                umma_f16(d, adesc + 2 * a_step, bdesc + 2 * adv_b, idesc, 1u);
                                umma_f16(d, adesc + 3 * a_step, bdesc + 3 * adv_b, idesc, 1u);
                            }
                        }
                        umma_commit(smem_u32(&empty_bar[stage]));
                    }
                    accw = 1u;
                    if (++stage == P.stages) {
                        stage = 0;
                        parity ^= 1;
                    }
                }
                if (!ok) break;
                if (elect_one()) {
                    if (nkb > 0) umma_commit(smem_u32(&tfull_bar[0]));
                    else mbar_arrive(smem_u32(&tfull_bar[0]));
                }
                continue;
            }
            if (!mbar_wait(smem_u32(&tempty_bar[buf]), tpar ^ 1, abort_flag, P.err, ERR_WAIT_TMEM_EMPTY)) {
                ok = false;
                break;
            }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + buf * P.bn;
            uint32_t acc = 0;
            if (kMode == MODE_FPROP && !kPair && P.patch) {
                int pp = 0;
                while (pp + 1 < P.n_phases && tile >= P.phases[pp + 1].tile_begin) ++pp;
                const Phase& ph = P.phases[pp];
                const uint32_t sbo_a = static_cast<uint32_t>(P.patch_w * P.a_stride_h) * 128u;  // 8-row groups: one output row = a_stride_h patch rows apart
                const uint64_t bdesc_ring0 = make_smem_desc(smem_u32(smem), lbo_b, b32 ? 512 : 1024, b32 ? 1 : 2);  // B ring starts the region
                for (int pass = 0; ok && pass < P.passes; ++pass)
                    for (int cb = 0; ok && cb < P.c_blocks; ++cb) {
                        if (!mbar_wait(smem_u32(&afull_bar[pstage]), pparity, abort_flag, P.err, ERR_WAIT_FULL)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        const uint32_t patch_addr = smem_u32(smem + P.a_ring_off) + pstage * P.patch_bytes;
                        const uint64_t adesc0 = make_smem_desc(patch_addr, 16, sbo_a, 2);
                        for (int t = 0; t < ph.tap_count; t += P.ka) {
                            if (!mbar_wait(smem_u32(&full_bar[stage]), parity, abort_flag, P.err, ERR_WAIT_FULL)) {
                                ok = false;
                                break;
                            }
                            tc_fence_after();
                            const int n = min(P.ka, ph.tap_count - t);
                            if (elect_one()) {
                                uint64_t bdesc = bdesc_ring0 + static_cast<uint64_t>(stage * P.ka * b_atom_step);
                                for (int j = 0; j < n; ++j) {
                                    const uint64_t adesc = adesc0 + static_cast<uint32_t>(P.taps[ph.tap_begin + t + j].aoff);
                                    if (f16) {
                                        umma_f16(d_tmem, adesc, bdesc, idesc, acc);
                                        umma_f16(d_tmem, adesc + 2, bdesc + adv_b, idesc, 1u);
                                        umma_f16(d_tmem, adesc + 4, bdesc + 2 * adv_b, idesc, 1u);
                                        umma_f16(d_tmem, adesc + 6, bdesc + 3 * adv_b, idesc, 1u);
                                    } else {
                                        umma_tf32(d_tmem, adesc, bdesc, idesc, acc);
                                        umma_tf32(d_tmem, adesc + 2, bdesc + adv_b, idesc, 1u);
                                        umma_tf32(d_tmem, adesc + 4, bdesc + 2 * adv_b, idesc, 1u);
                                        umma_tf32(d_tmem, adesc + 6, bdesc + 3 * adv_b, idesc, 1u);
                                    }
                                    acc = 1u;
                                    bdesc += b_atom_step;
                                }
                                umma_commit(smem_u32(&empty_bar[stage]));
                            }
                            acc = 1u;
                            if (++stage == P.stages) {
                                stage = 0;
                                parity ^= 1;
                            }
                        }
                        if (!ok) break;
                        if (elect_one()) umma_commit(smem_u32(&aempty_bar[pstage]));
                        if (++pstage == P.a_stages) {
                            pstage = 0;
                            pparity ^= 1;
                        }
                    }
            } else
            for (int it = 0; it < k_iters; it += P.ka) {
                const int n_atoms = min(P.ka, k_iters - it);
                if (!mbar_wait(smem_u32(&full_bar[stage]), parity, abort_flag, P.err, ERR_WAIT_FULL)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                if (elect_one()) {  // elect.sync keeps the issue path on the uniform datapath
                    uint64_t adesc = adesc0 + static_cast<uint64_t>(stage * stage_step);
                    uint64_t bdesc = bdesc0 + static_cast<uint64_t>(stage * stage_step);
                    uint32_t first = acc;
                    for (int a = 0; a < n_atoms; ++a) {
                        if (kPair) {
                            if (f16) {
                                umma_f16_pair(d_tmem, adesc, bdesc, idesc, first);
                                umma_f16_pair(d_tmem, adesc + adv_a, bdesc + adv_b, idesc, 1u);
                                umma_f16_pair(d_tmem, adesc + 2 * adv_a, bdesc + 2 * adv_b, idesc, 1u);
                                umma_f16_pair(d_tmem, adesc + 3 * adv_a, bdesc + 3 * adv_b, idesc, 1u);
                            } else {
                                umma_tf32_pair(d_tmem, adesc, bdesc, idesc, first);
                                umma_tf32_pair(d_tmem, adesc + adv_a, bdesc + adv_b, idesc, 1u);
                                umma_tf32_pair(d_tmem, adesc + 2 * adv_a, bdesc + 2 * adv_b, idesc, 1u);
                                umma_tf32_pair(d_tmem, adesc + 3 * adv_a, bdesc + 3 * adv_b, idesc, 1u);
                            }
                        } else if (f16) {
                            umma_f16(d_tmem, adesc, bdesc, idesc, first);
                            umma_f16(d_tmem, adesc + adv_a, bdesc + adv_b, idesc, 1u);
                            umma_f16(d_tmem, adesc + 2 * adv_a, bdesc + 2 * adv_b, idesc, 1u);
                            umma_f16(d_tmem, adesc + 3 * adv_a, bdesc + 3 * adv_b, idesc, 1u);
                        } else {
                            umma_tf32(d_tmem, adesc, bdesc, idesc, first);
                            umma_tf32(d_tmem, adesc + adv_a, bdesc + adv_b, idesc, 1u);
                            umma_tf32(d_tmem, adesc + 2 * adv_a, bdesc + 2 * adv_b, idesc, 1u);
                            umma_tf32(d_tmem, adesc + 3 * adv_a, bdesc + 3 * adv_b, idesc, 1u);
                        }
                        first = 1u;
                        adesc += a_atom_step;
                        bdesc += b_atom_step;
                    }
                    if (kPair) umma_commit_pair(smem_u32(&empty_bar[stage]));  // frees the stage in both CTAs
                    else umma_commit(smem_u32(&empty_bar[stage]));
                }
                acc = 1u;
                if (++stage == P.stages) {
                    stage = 0;
                    parity ^= 1;
                }
            }
            if (!ok) break;
            if (elect_one()) {
                if (kPair) {
                    if (k_iters > 0) {
                        umma_commit_pair(smem_u32(&tfull_bar[buf]));
                    } else {
                        mbar_arrive(smem_u32(&tfull_bar[buf]));
                        mbar_arrive_cluster(map_to_cta(smem_u32(&tfull_bar[buf]), 1));
                    }
                } else if (k_iters > 0)
                    umma_commit(smem_u32(&tfull_bar[buf]));
                else
                    mbar_arrive(smem_u32(&tfull_bar[buf]));
            }
        }
    }
    // ------------------------------------------------------------ epilogue --
    else if (warp < 6 || P.epi_warps == 8) {
        const int ew = (warp < 6) ? warp - 2 : warp - 3;  // epilogue warp index 0..7; 4..7 form the second group
        const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
        const int row = quarter * 32 + lane;
        bool ok = true;
        int titer = 0;
        uint32_t store_seq = 0;  // TMA-store pieces issued by this warp so far (selects the staging buffer)
        int bias_ntile = -1;     // column tile whose bias values sit in this warp's shared-memory copy
        for (int tile_id = tile_first; ok && tile_id < P.num_tiles; tile_id += tile_step, ++titer) {
            int tile = tile_id, kz = 0;
            if (kMode == MODE_FPROP && P.fsplit > 1) {
                kz = tile_id / P.base_tiles;
                tile = tile_id - kz * P.base_tiles;
            }
            if (kMode == MODE_WGRAD && !kPair && P.wpatch) {
                // patch walk: every row tile of the gradient sits in TMEM, accumulator i in columns [i*bn, (i+1)*bn)
                const int w_ntile = tile % P.n_tiles, w_z = tile / P.n_tiles;
                const int per = (P.kblocks_total + P.split_k - 1) / P.split_k;
                const int nkb = max(min(w_z * per + per, P.kblocks_total) - w_z * per, 0);
                if (!mbar_wait(smem_u32(&tfull_bar[0]), titer & 1, abort_flag, P.err, ERR_WAIT_TMEM_FULL)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const int w_col_base = w_ntile * P.bn;
                // this K slice's plane of the partial gradient (laid out like dW itself)
                float* const w_plane = reinterpret_cast<float*>(P.out) + static_cast<size_t>(w_z) * P.plane_elems;
                const bool w_live = nkb > 0;  // an empty slice stores zeros (its accumulators were never written)
                if (P.w_coalesce) {
                    // A column of the gradient (one channel of the other tensor) is ONE contiguous run of
                    // c_patch * taps floats in memory, and 32 columns are 32 such runs back to back.  Scattering the
                    // accumulators' rows straight into them costs a 32-sector store per instruction; instead the
                    // four warps lay 32 columns out in shared memory (the operand ring is idle by now: this CTA has
                    // no further tile) and store them as contiguous 128-byte pieces.
                    float* S = reinterpret_cast<float*>(smem);
                    const size_t run = static_cast<size_t>(P.c_patch) * P.n_taps * (P.kw_pack ? P.kw_count : 1);
                    uint32_t syncs = 0;
                    auto meet = [&]() -> bool {  // bounded meeting of the four epilogue warps
                        __syncwarp();
                        const uint32_t bar = smem_u32(&afull_bar[syncs & 1]);
                        if (lane == 0) mbar_arrive(bar);
                        const bool met = mbar_wait(bar, (syncs >> 1) & 1, abort_flag, P.err, ERR_WAIT_TMEM_FULL);
                        ++syncs;
                        return met;
                    };
                    fence_proxy_async();
                    for (int c0 = 0; ok && c0 < P.bn; c0 += 32) {
                        const int cg = w_col_base + c0;
                        if (cg >= P.c_out) break;  // uniform across the CTA
                        const int ncols = min(32, P.c_out - cg);
#pragma unroll 1
                        for (int i = 0; i < P.w_mtiles; ++i) {
                            const int gi = i * (kTileM / P.kb) + row / P.kb;
                            const int pc = row % P.kb;
                            bool w_valid;
                            size_t w_off;
                            if (P.kw_pack) {
                                const int kwi = pc >> 3, c = pc & 7;
                                w_valid = (gi < P.groups_total) && (c < P.c_patch) && (kwi < P.kw_count);
                                w_off = (static_cast<size_t>(c) * P.n_taps + gi) * P.kw_count + kwi;
                            } else {
                                w_valid = (gi < P.groups_total) && (pc < P.c_patch);
                                w_off = static_cast<size_t>(pc) * P.n_taps + gi;
                            }
                            uint32_t r[32];
                            tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + i * P.bn + c0, r);
                            tmem_ld_wait();
                            if (w_valid) {
#pragma unroll
                                for (int j = 0; j < 32; ++j)
                                    if (j < ncols) S[j * run + w_off] = w_live ? __uint_as_float(r[j]) : 0.f;
                            }
                            __syncwarp();
                        }
                        if (!meet()) {
                            ok = false;
                            break;
                        }
                        float* o = w_plane + static_cast<size_t>(cg) * run;
                        const size_t total = static_cast<size_t>(ncols) * run;
                        for (size_t idx = static_cast<size_t>(ew) * 32 + lane; idx < total; idx += 128) o[idx] = S[idx];
                        if (!meet()) {  // the next 32 columns overwrite S
                            ok = false;
                            break;
                        }
                    }
                    if (!ok) break;
                } else
#pragma unroll 1
                for (int i = 0; i < P.w_mtiles; ++i) {
                    const int gi = i * (kTileM / P.kb) + row / P.kb;  // tap (kernel row with kw packing) of this row
                    const int pc = row % P.kb;
                    bool w_valid;
                    size_t w_off, w_stride;
                    if (P.kw_pack) {
                        const int kwi = pc >> 3, c = pc & 7;
                        w_valid = (gi < P.groups_total) && (c < P.c_patch) && (kwi < P.kw_count);
                        w_off = (static_cast<size_t>(c) * P.n_taps + gi) * P.kw_count + kwi;
                        w_stride = static_cast<size_t>(P.c_patch) * P.n_taps * P.kw_count;
                    } else {
                        w_valid = (gi < P.groups_total) && (pc < P.c_patch);
                        w_off = static_cast<size_t>(pc) * P.n_taps + gi;
                        w_stride = static_cast<size_t>(P.c_patch) * P.n_taps;
                    }
                    const uint32_t w_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + i * P.bn;
                    for (int c0 = 0; c0 < P.bn; c0 += 32) {
                        if (w_col_base + c0 >= P.c_out) break;  // uniform across the warp
                        uint32_t r[32];
                        tmem_ld_32x32(w_row + c0, r);
                        tmem_ld_wait();
                        const int cg = w_col_base + c0;
                        const int ncols = min(32, P.c_out - cg);
                        if (w_valid) {
                            float* o = w_plane + w_off + static_cast<size_t>(cg) * w_stride;
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (j < ncols) o[j * w_stride] = w_live ? __uint_as_float(r[j]) : 0.f;
                        }
                        __syncwarp();  // tcgen05.ld is warp-collective: reconverge before the next chunk
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[0]));
                continue;
            }
            const int buf = titer & 1;
            const uint32_t tpar = (titer >> 1) & 1;
            // tile decode
            int ntile, k_iters;
            bool row_valid;
            int pix_n = 0, pix_h = 0, pix_w = 0;  // forward walk: this row's pixel within its phase grid
            size_t row_off = 0;     // NHWC / wgrad: element offset of column 0; NCHW: pixel offset
            size_t col_stride = 1;  // element distance between consecutive columns
            int kslice = kz;        // K slice of this tile (K-split forward walk, split-K weight gradient)
            if (kMode == MODE_FPROP) {
                int p = 0;
                while (p + 1 < P.n_phases && tile >= P.phases[p + 1].tile_begin) ++p;
                const Phase& ph = P.phases[p];
                int local = tile - ph.tile_begin;
                int tw, th, tn;
                decode_fprop_tile<kPair>(P, ph, local, cta_rank, ntile, tw, th, tn);
                int iw = (tw << P.wb_log2) + (row & (wb - 1));
                int ih = (th << P.hb_log2) + ((row >> P.wb_log2) & (hb - 1));
                int n = (tn << P.nb_log2) + (row >> (P.wb_log2 + P.hb_log2));
                row_valid = (iw < ph.wq) && (ih < ph.hq) && (n < P.batch);
                pix_n = n;
                pix_h = ih;
                pix_w = iw;
                int ow = ph.pw + P.out_stride_w * iw;
                int oh = ph.ph + P.out_stride_h * ih;
                k_iters = ph.tap_count;
                if (P.fsplit > 1) {  // K iterations of this slice (0: nothing to add)
                    const int full = P.passes * ph.tap_count * P.c_blocks;
                    const int per = (full + P.fsplit - 1) / P.fsplit;
                    const int k_first = min(kz * per, full);
                    k_iters = min(k_first + per, full) - k_first;
                }
                if (kOutMode != OUT_NCHW && kOutMode != OUT_NCHW_TMA) {
                    row_off = ((static_cast<size_t>(n) * P.out_h + oh) * P.out_w + ow) * P.ld_out;
                    col_stride = 1;
                } else {
                    row_off = (static_cast<size_t>(n) * P.c_out * P.out_h + oh) * P.out_w + ow;
                    col_stride = static_cast<size_t>(P.out_h) * P.out_w;
                }
            } else {
                int m_tiles = (P.groups_total * P.kb + kTileM - 1) / kTileM;
                if (kPair) m_tiles = (m_tiles + 1) / 2;  // tile ids name pairs of row tiles
                int mt, z;
                decode_wgrad_tile(P, tile, m_tiles, ntile, mt, z);
                if (kPair) mt = 2 * mt + static_cast<int>(cta_rank);
                int per = (P.kblocks_total + P.split_k - 1) / P.split_k;
                k_iters = max(min(z * per + per, P.kblocks_total) - z * per, 0);
                kslice = z;
                int gi = mt * (kTileM / P.kb) + row / P.kb;
                int t = gi / P.c_blocks;
                int cib = gi - t * P.c_blocks;
                int pc = cib * P.kb + (row % P.kb);
                if (P.kw_pack) {
                    // few-channel path: tap t is a kernel row kh, patch index pc packs (kw, c)
                    const int kwi = pc >> 3, c = pc & 7;
                    row_valid = (gi < P.groups_total) && (c < P.c_patch) && (kwi < P.kw_count);
                    row_off = (static_cast<size_t>(c) * P.n_taps + t) * P.kw_count + kwi;
                    col_stride = static_cast<size_t>(P.c_patch) * P.n_taps * P.kw_count;
                } else {
                    row_valid = (gi < P.groups_total) && (pc < P.c_patch);
                    // dW[plain][patch][tap]
                    row_off = static_cast<size_t>(pc) * P.n_taps + t;
                    col_stride = static_cast<size_t>(P.c_patch) * P.n_taps;
                }
                if (P.split_k > 1) {
                    // partial sums go to this slice's plane, [column][row of the tile walk]: lanes are consecutive
                    // rows, so every column store coalesces; rows beyond the gradient are written too (the planes
                    // are padded to whole tiles) and never read
                    row_valid = true;
                    row_off = static_cast<size_t>(mt) * kTileM + row;
                    col_stride = static_cast<size_t>(P.ld_plane);
                }
            }
            if (kMode == MODE_FPROP && NML_IS_TMA_OUT(kOutMode) && P.bias != nullptr) {
                // this tile's bias values, one copy per warp (no cross-warp barrier to get stuck on)
                // (skipped when the column tile is the one this warp loaded last; all eight loads of a lane are
                // issued before the first is used, so the fill costs one memory latency, not eight)
                if (ntile != bias_ntile) {
                    bias_ntile = ntile;
                    float* btw = bias_tile + ew * 256;
                    const int cb0 = ntile * P.bn;
                    float bv[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int j = lane + 32 * u;
                        bv[u] = !(j < P.bn && cb0 + j < P.c_out) ? 0.f
                                : P.bias_f16 ? __half2float(__ldg(reinterpret_cast<const __half*>(P.bias) + cb0 + j))
                                             : __ldg(P.bias + cb0 + j);
                    }
                    __syncwarp();
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        if (lane + 32 * u < P.bn) btw[lane + 32 * u] = bv[u];
                    __syncwarp();
                }
            }
            // Row-major epilogue: this lane's bias slice for the first 128-byte piece is fetched before
            // the wait, and each later slice one piece ahead, so the load latency never shows.
            float4 nb0 = make_float4(0.f, 0.f, 0.f, 0.f), nb1 = nb0;
            if (kMode == MODE_FPROP && kOutMode == OUT_NHWC && P.bias != nullptr &&
                (reinterpret_cast<uintptr_t>(P.bias) & 15) == 0) {
                const int cpi0 = kOutF16 ? 64 : 32;
                const int cgf = ntile * P.bn;
                if (cgf + cpi0 <= P.c_out) {
                    const int ql = lane & 7;
                    if (kOutF16) {
                        nb0 = __ldg(reinterpret_cast<const float4*>(P.bias + cgf + 8 * ql));
                        nb1 = __ldg(reinterpret_cast<const float4*>(P.bias + cgf + 8 * ql + 4));
                    } else {
                        nb0 = __ldg(reinterpret_cast<const float4*>(P.bias + cgf + 4 * ql));
                    }
                }
            }
            if (!mbar_wait(smem_u32(&tfull_bar[buf]), tpar, abort_flag, P.err, ERR_WAIT_TMEM_FULL)) {
                ok = false;
                break;
            }
            tc_fence_after();
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * P.bn;
            const int col_base = ntile * P.bn;
            if (kMode == MODE_FPROP && NML_IS_TMA_OUT(kOutMode)) {
                // Row-major output through TMA: each warp converts 128-byte row pieces of its 32 rows into a
                // swizzled 4 KB buffer and one lane hands the buffer to a TMA store, whose box is exactly
                // those 32 rows; rows and columns outside the tensor are clipped by the hardware.  Two
                // buffers alternate, so packing the next piece overlaps the store of the previous one.
                constexpr int cpi = kOutF16 ? 64 : 32;
                const uint32_t stg0 = smem_u32(staging) + ew * P.stg_bufs * kStagingBufBytes;
                const float* bt = bias_tile + ew * 256;
                const bool has_bias = (P.bias != nullptr);
                // store coordinates of this warp's first row
                int sw, sh, sn;
                {
                    int p = 0;
                    while (p + 1 < P.n_phases && tile >= P.phases[p + 1].tile_begin) ++p;
                    const Phase& ph = P.phases[p];
                    int local = tile - ph.tile_begin;
                    int nt_unused, tw, th, tn;
                    decode_fprop_tile<kPair>(P, ph, local, cta_rank, nt_unused, tw, th, tn);
                    const int row0 = quarter * 32;
                    sw = ph.pw + P.out_stride_w * ((tw << P.wb_log2) + (row0 & (wb - 1)));
                    sh = ph.ph + P.out_stride_h * ((th << P.hb_log2) + ((row0 >> P.wb_log2) & (hb - 1)));
                    sn = (tn << P.nb_log2) + (row0 >> (P.wb_log2 + P.hb_log2));
                }
                uint32_t r0[32], r1[32];
                const bool live = (k_iters > 0);
                if (!live) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) r0[j] = r1[j] = 0u;
                }
                // with two epilogue groups, the first takes the low half of the tile's pieces, the second the rest
                int c_begin = 0, c_end = P.bn;
                if (P.epi_warps == 8) {
                    const int half = ((P.bn / cpi + 1) / 2) * cpi;
                    if (ew < 4) c_end = min(half, P.bn); else c_begin = half;
                }
                if (live && c_begin < c_end && col_base + c_begin < P.c_out) {
                    tmem_ld_32x32(t_row + c_begin, r0);
                    if (cpi == 64) tmem_ld_32x32(t_row + c_begin + 32, r1);
                    tmem_ld_wait();
                }
                for (int c0 = c_begin; c0 < c_end; c0 += cpi) {
                    const int cg = col_base + c0;
                    if (cg >= P.c_out) break;  // uniform across the warp
                    const int cn = c0 + cpi;
                    const bool more = live && cn < c_end && col_base + cn < P.c_out;
                    const uint32_t buf_addr = stg0 + ((P.stg_bufs == 2) ? (store_seq & 1) * kStagingBufBytes : 0);
                    // the store that last read this buffer must be done reading it
                    if (lane == 0) {
                        if (P.stg_bufs == 2) bulk_wait_group_read<1>(); else bulk_wait_group_read<0>();
                    }
                    __syncwarp();
                    if (kOutMode == OUT_NCHW_TMA) {
                        // channel-major output: the staging tile is [image][channel][h][w] of this warp's
                        // pixel sub-box, so lane (= pixel) l writes channel j at ((dn*cpi + j)*bh + dh)*bw + dw
                        const int bwl = P.cm_bw_log2, bhl = P.cm_bh_log2;
                        const int dwp = lane & ((1 << bwl) - 1);
                        const int dhp = (lane >> bwl) & ((1 << bhl) - 1);
                        const int dnp = lane >> (bwl + bhl);
                        const uint32_t esz = kOutF16 ? 2 : 4;
                        const uint32_t pix = buf_addr + ((((dnp * cpi) << bhl) + dhp) << bwl) * esz + dwp * esz;
                        const uint32_t cstep = (esz << (bwl + bhl));  // bytes between consecutive channels
#pragma unroll
                        for (int j = 0; j < cpi; ++j) {
                            float xv = __uint_as_float(j < 32 ? r0[j & 31] : r1[j & 31]);
                            if (has_bias) xv += bt[c0 + j];
                            if (kOutF16) {
                                const __half hv = __float2half_rn(xv);
                                asm volatile("st.shared.b16 [%0], %1;" ::"r"(pix + j * cstep), "h"(*reinterpret_cast<const uint16_t*>(&hv)) : "memory");
                            } else {
                                if (P.round_f16) xv = round_through_f16(xv);
                                asm volatile("st.shared.b32 [%0], %1;" ::"r"(pix + j * cstep), "r"(__float_as_uint(xv)) : "memory");
                            }
                        }
                    } else
#pragma unroll
                    for (int qq = 0; qq < 8; ++qq) {
                        uint4 pk;
                        if (kOutF16) {
                            const uint32_t* src = (qq < 4) ? &r0[8 * qq] : &r1[8 * (qq - 4)];
                            float v[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(src[j]);
                            if (has_bias) {
                                const float4 ba = *reinterpret_cast<const float4*>(bt + c0 + 8 * qq);
                                const float4 bb = *reinterpret_cast<const float4*>(bt + c0 + 8 * qq + 4);
                                v[0] += ba.x; v[1] += ba.y; v[2] += ba.z; v[3] += ba.w;
                                v[4] += bb.x; v[5] += bb.y; v[6] += bb.z; v[7] += bb.w;
                            }
                            pk.x = pack_half2(v[0], v[1]);
                            pk.y = pack_half2(v[2], v[3]);
                            pk.z = pack_half2(v[4], v[5]);
                            pk.w = pack_half2(v[6], v[7]);
                        } else {
                            float v[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) v[j] = __uint_as_float(r0[4 * qq + j]);
                            if (has_bias) {
                                const float4 ba = *reinterpret_cast<const float4*>(bt + c0 + 4 * qq);
                                v[0] += ba.x; v[1] += ba.y; v[2] += ba.z; v[3] += ba.w;
                            }
                            if (P.round_f16) {
#pragma unroll
                                for (int j = 0; j < 4; ++j) v[j] = round_through_f16(v[j]);
                            }
                            pk.x = __float_as_uint(v[0]); pk.y = __float_as_uint(v[1]);
                            pk.z = __float_as_uint(v[2]); pk.w = __float_as_uint(v[3]);
                        }
                        st_shared_v4(buf_addr + lane * 128 + ((qq ^ (lane & 7)) << 4), pk);
                    }
                    if (more) {  // registers are free again: start the next TMEM load now
                        tmem_ld_32x32(t_row + cn, r0);
                        if (cpi == 64) tmem_ld_32x32(t_row + cn + 32, r1);
                    }
                    fence_proxy_async();  // make the generic-proxy writes visible to the TMA engine
                    __syncwarp();
                    if (lane == 0) {
                        if (kOutMode == OUT_NCHW_TMA) tma_store_4d(&P.tmC, buf_addr, sw, sh, cg, sn);
                        else tma_store_4d(&P.tmC, buf_addr, cg, sw, sh, sn);
                        bulk_commit_group();
                    }
                    ++store_seq;
                    if (more) tmem_ld_wait();
                }
            } else
            if (kMode == MODE_FPROP && kOutMode == OUT_NHWC && P.shuf_sh > 0) {
                // Phase-packed columns: this thread's pixel owns shuf_sh rows of shuf_sw * shuf_c consecutive
                // output values.  Short on purpose, like the few-channel epilogue below.
                uint32_t r[16];
                if (k_iters > 0) {
                    tmem_ld_32x16(t_row, r);
                    tmem_ld_wait();
                }
                if (row_valid) {
                    const int run = P.shuf_sw * P.shuf_c;
                    const int ow0 = P.shuf_sw * pix_w;
                    const int oh0 = P.shuf_sh * pix_h;
                    // column j = (phs, pw, c), walked with counters (no divisions in the unrolled body)
                    int phs = 0, q = 0, pw = 0, cc = 0;
                    size_t o_row = ((static_cast<size_t>(pix_n) * P.shuf_oh + oh0) * P.shuf_ow + ow0) * P.shuf_c;
                    const size_t o_step = static_cast<size_t>(P.shuf_ow) * P.shuf_c;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (j < P.c_out) {
                            if (oh0 + phs < P.shuf_oh && ow0 + pw < P.shuf_ow) {
                                float xv = (k_iters > 0) ? __uint_as_float(r[j]) : 0.f;
                                if (P.bias != nullptr) xv += __ldg(P.bias + j);
                                if (kOutF16) {
                                    reinterpret_cast<__half*>(P.out)[o_row + q] = __float2half_rn(xv);
                                } else {
                                    if (P.round_f16) xv = round_through_f16(xv);
                                    reinterpret_cast<float*>(P.out)[o_row + q] = xv;
                                }
                            }
                            if (++cc == P.shuf_c) {
                                cc = 0;
                                ++pw;
                            }
                            if (++q == run) {
                                q = 0;
                                pw = 0;
                                ++phs;
                                o_row += o_step;
                            }
                        }
                    }
                }
            } else
            if (kMode == MODE_FPROP && kOutMode == OUT_NHWC && P.c_out <= 8 && P.fsplit <= 1) {
                // A handful of output channels (image-producing layers, input gradients of stems): each
                // thread stores its pixel's few values.  Kept short on purpose -- the epilogue warps are
                // bound by instruction fetch, not by the stores.
                uint32_t r[8];
                if (k_iters > 0) {
                    tmem_ld_32x8(t_row, r);
                    tmem_ld_wait();
                }
                if (row_valid) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (j < P.c_out) {
                            float xv = (k_iters > 0) ? __uint_as_float(r[j]) : 0.f;
                            if (P.bias != nullptr) xv += __ldg(P.bias + j);
                            if (kOutF16) {
                                reinterpret_cast<__half*>(P.out)[row_off + j] = __float2half_rn(xv);
                            } else {
                                if (P.round_f16) xv = round_through_f16(xv);
                                reinterpret_cast<float*>(P.out)[row_off + j] = xv;
                            }
                        }
                    }
                }
            } else
            if (kMode == MODE_FPROP && kOutMode == OUT_NHWC && P.fsplit <= 1) {
                // Row-major output.  Each 128-byte piece of a row (64 fp16 / 32 fp32 columns) goes
                // through a swizzled shared-memory tile so that a warp store writes four full
                // 128-byte row pieces instead of 32 scattered 16-byte ones.  The TMEM load of the
                // next piece is in flight while the current one is written out, and the bias is
                // added on the way out, where each lane owns the same 16 bytes of every row.
                const int cpi = kOutF16 ? 64 : 32;
                const int esz = kOutF16 ? 2 : 4;
                const uint32_t stg = smem_u32(staging) + ew * P.stg_bufs * kStagingBufBytes;
                const bool has_bias = (P.bias != nullptr);
                const bool aligned = ((static_cast<size_t>(P.ld_out) * esz) & 15) == 0 &&
                                     (reinterpret_cast<uintptr_t>(P.out) & 15) == 0 &&
                                     (reinterpret_cast<uintptr_t>(P.bias) & 15) == 0;
                // rows this lane writes out: rr = it*4 + lane/8
                unsigned long long my_off[8];
                uint32_t my_ok = 0;
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    const int rr = it * 4 + (lane >> 3);
                    my_off[it] = __shfl_sync(0xffffffffu, static_cast<unsigned long long>(row_off), rr);
                    my_ok |= (__shfl_sync(0xffffffffu, row_valid ? 1u : 0u, rr) & 1u) << it;
                }
                const int q = lane & 7;
                uint8_t* obase = reinterpret_cast<uint8_t*>(P.out);
                uint32_t r0[32], r1[32];
                const bool live = (k_iters > 0);
                if (!live) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) r0[j] = r1[j] = 0u;
                }
                if (live && col_base < P.c_out) {
                    tmem_ld_32x32(t_row, r0);
                    if (cpi == 64 && 32 < P.bn) tmem_ld_32x32(t_row + 32, r1);
                    tmem_ld_wait();
                }
                for (int c0 = 0; c0 < P.bn; c0 += cpi) {
                    const int cg = col_base + c0;
                    if (cg >= P.c_out) break;  // uniform across the warp
                    const int ncols = min(min(cpi, P.bn - c0), P.c_out - cg);
                    const int cn = c0 + cpi;   // next piece
                    const bool more = live && cn < P.bn && col_base + cn < P.c_out;
                    if (ncols == cpi && aligned) {
#pragma unroll
                        for (int qq = 0; qq < 8; ++qq) {
                            uint4 pk;
                            if (kOutF16) {
                                const uint32_t* src = (qq < 4) ? &r0[8 * qq] : &r1[8 * (qq - 4)];
                                pk.x = pack_half2(__uint_as_float(src[0]), __uint_as_float(src[1]));
                                pk.y = pack_half2(__uint_as_float(src[2]), __uint_as_float(src[3]));
                                pk.z = pack_half2(__uint_as_float(src[4]), __uint_as_float(src[5]));
                                pk.w = pack_half2(__uint_as_float(src[6]), __uint_as_float(src[7]));
                            } else {
                                pk.x = r0[4 * qq]; pk.y = r0[4 * qq + 1]; pk.z = r0[4 * qq + 2]; pk.w = r0[4 * qq + 3];
                            }
                            st_shared_v4(stg + lane * 128 + ((qq ^ (lane & 7)) << 4), pk);
                        }
                        if (more) {  // registers are free again: start the next TMEM load now
                            tmem_ld_32x32(t_row + cn, r0);
                            if (cpi == 64 && cn + 32 < P.bn) tmem_ld_32x32(t_row + cn + 32, r1);
                        }
                        __syncwarp();
                        // this lane's slice of the bias: columns cg + q*8 .. +7 (fp16) or cg + q*4 .. +3 (fp32)
                        const float4 b0 = nb0, b1 = nb1;
                        if (has_bias) {  // fetch the next piece's slice now; it is used one piece later
                            const int cgn = cg + cpi;
                            if (c0 + cpi < P.bn && cgn + cpi <= P.c_out) {
                                if (kOutF16) {
                                    nb0 = __ldg(reinterpret_cast<const float4*>(P.bias + cgn + 8 * q));
                                    nb1 = __ldg(reinterpret_cast<const float4*>(P.bias + cgn + 8 * q + 4));
                                } else {
                                    nb0 = __ldg(reinterpret_cast<const float4*>(P.bias + cgn + 4 * q));
                                }
                            }
                        }
                        const __half2 hb0 = __floats2half2_rn(b0.x, b0.y), hb1 = __floats2half2_rn(b0.z, b0.w);
                        const __half2 hb2 = __floats2half2_rn(b1.x, b1.y), hb3 = __floats2half2_rn(b1.z, b1.w);
#pragma unroll
                        for (int it = 0; it < 8; ++it) {
                            const int rr = it * 4 + (lane >> 3);
                            uint4 pk = ld_shared_v4(stg + rr * 128 + ((q ^ (rr & 7)) << 4));
                            if (has_bias) {
                                if (kOutF16) {
                                    // fp16 add on the fp16-rounded product, as the reference's bias kernel does
                                    __half2 h;
                                    h = __hadd2(*reinterpret_cast<__half2*>(&pk.x), hb0); pk.x = *reinterpret_cast<uint32_t*>(&h);
                                    h = __hadd2(*reinterpret_cast<__half2*>(&pk.y), hb1); pk.y = *reinterpret_cast<uint32_t*>(&h);
                                    h = __hadd2(*reinterpret_cast<__half2*>(&pk.z), hb2); pk.z = *reinterpret_cast<uint32_t*>(&h);
                                    h = __hadd2(*reinterpret_cast<__half2*>(&pk.w), hb3); pk.w = *reinterpret_cast<uint32_t*>(&h);
                                } else {
                                    pk.x = __float_as_uint(__uint_as_float(pk.x) + b0.x);
                                    pk.y = __float_as_uint(__uint_as_float(pk.y) + b0.y);
                                    pk.z = __float_as_uint(__uint_as_float(pk.z) + b0.z);
                                    pk.w = __float_as_uint(__uint_as_float(pk.w) + b0.w);
                                }
                            }
                            if (!kOutF16 && P.round_f16) {
                                pk.x = __float_as_uint(round_through_f16(__uint_as_float(pk.x)));
                                pk.y = __float_as_uint(round_through_f16(__uint_as_float(pk.y)));
                                pk.z = __float_as_uint(round_through_f16(__uint_as_float(pk.z)));
                                pk.w = __float_as_uint(round_through_f16(__uint_as_float(pk.w)));
                            }
                            if ((my_ok >> it) & 1u)
                                *reinterpret_cast<uint4*>(obase + (my_off[it] + cg) * esz + q * 16) = pk;
                        }
                        __syncwarp();
                        if (more) tmem_ld_wait();
                    } else {
                        // ragged tail or unaligned rows: per-thread stores, 32 columns at a time
#pragma unroll 1
                        for (int half = 0; half < 2; ++half) {
                            const int cgh = cg + half * 32;
                            const int nh = min(32, ncols - half * 32);
                            if (nh <= 0) break;
                            float v[32];
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                float xv = __uint_as_float(half == 0 ? r0[j] : r1[j]);
                                if (has_bias && j < nh) xv += P.bias[cgh + j];
                                if (P.round_f16) xv = round_through_f16(xv);
                                v[j] = xv;
                            }
                            if (row_valid) store_row_chunk(P, v, row_off, col_stride, cgh, nh);
                        }
                        __syncwarp();
                        if (more) {
                            tmem_ld_32x32(t_row + cn, r0);
                            if (cpi == 64 && cn + 32 < P.bn) tmem_ld_32x32(t_row + cn + 32, r1);
                            tmem_ld_wait();
                        }
                    }
                }
            } else
            for (int c0 = 0; c0 < P.bn; c0 += 32) {
                if (col_base + c0 >= P.c_out) break;  // uniform across the warp
                uint32_t r[32];
                if (k_iters > 0) {
                    tmem_ld_32x32(t_row + c0, r);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] = 0u;
                }
                const int cg = col_base + c0;
                const int ncols = min(32, P.c_out - cg);
                if (kMode == MODE_WGRAD || (kOutMode == OUT_NHWC && P.fsplit > 1)) {
                    // the gradient itself (one K slice) or this K slice's plane of partial sums; an empty
                    // slice stores the zeros loaded above
                    if (row_valid) {
                        float* o = reinterpret_cast<float*>(P.out) + static_cast<size_t>(kslice) * P.plane_elems + row_off +
                                   static_cast<size_t>(cg) * col_stride;
                        if (kMode == MODE_FPROP && ncols == 32 && (P.ld_out & 3) == 0) {
#pragma unroll
                            for (int q = 0; q < 8; ++q)
                                reinterpret_cast<float4*>(o)[q] = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                                                              __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (j < ncols) o[j * col_stride] = __uint_as_float(r[j]);
                        }
                    }
                } else {
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        float x = __uint_as_float(r[j]);
                        if (P.bias != nullptr && j < ncols) x += P.bias[cg + j];
                        if (P.round_f16) x = round_through_f16(x);
                        v[j] = x;
                    }
                    if (row_valid) store_row_chunk(P, v, row_off, col_stride, cg, ncols);
                }
                __syncwarp();  // tcgen05.ld is warp-collective: reconverge before the next chunk
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (kPair && !leader) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[buf]), 0));
                else mbar_arrive(smem_u32(&tempty_bar[buf]));
            }
        }
        if (NML_IS_TMA_OUT(kOutMode) && lane == 0) bulk_wait_group<0>();  // stores must land before the CTA ends
    }

    // ------------------------------------------------------------ teardown --
    tc_fence_before();
    __syncthreads();
    if (kPair) cluster_sync_all();  // neither CTA may leave (or free TMEM) while the partner can still touch it
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        if (kPair) tmem_dealloc_pair(tmem_base, tmem_cols);
        else tmem_dealloc(tmem_base, tmem_cols);
    }
}

}  // namespace nml

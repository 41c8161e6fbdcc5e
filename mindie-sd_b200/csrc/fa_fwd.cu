// Flash-attention forward for sm_100a: tcgen05 MMA into tensor memory, TMA-staged operands,
// warp-specialised roles, online softmax.  One kernel serves dense and block-sparse attention
// (bf16 / fp16 operands) and the e4m3-quantised variant.
//
// Work decomposition.  One CTA owns a pair of 128-row query tiles of one (batch, head) and walks
// the 128-row key/value blocks either tile attends to.  Per tile the score block S = Q K^T lives
// in 128 fp32 columns of tensor memory, the probabilities P overwrite the front of those columns
// in operand precision, and the output accumulator O holds another 128 columns:
//     columns   0..127  S0 / P0      128..255  S1 / P1      256..383  O0      384..511  O1
// Roles (12 warps, the last two idle so that every scheduler partition holds three):
//     warps 0-3   softmax + O rescale + epilogue of tile 0 (one query row per thread)
//     warps 4-7   the same for tile 1
//     warp  8     MMA issue (one thread)
//     warp  9     TMA loads (one thread)
// The MMA thread interleaves the two tiles (S0, S1, PV0, S0', PV1, S1', ...) so the tensor pipe
// has work of one tile while the other tile's rows are in the exponent unit.
#include "fa_fwd.h"
#include "ptx_sm100.cuh"
#include "rf_grid.cuh"

#include <cuda_bf16.h>
#include <type_traits>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

// Development aid, off in every shipped build: with -DSDB_FA_TRACE one thread block records clock64()
// stamps of its roles for key blocks 200..231 into the buffer passed as `lse` (which is then not
// written as a log-sum-exp): [role][block - 200][slot], role 0/1 = softmax of tile 0/1, 2 = MMA thread.
#ifdef SDB_FA_TRACE
#define SDB_TR(role, idx, slot)                                                                                  \
    do {                                                                                                         \
        if (blockIdx.x == 40 && blockIdx.y == 0 && blockIdx.z == 0 && p.lse != nullptr && (idx) >= 200 && (idx) < 232) \
            reinterpret_cast<long long*>(p.lse)[((role) * 32 + ((idx) - 200)) * 16 + (slot)] = clock64();          \
    } while (0)
#else
#define SDB_TR(role, idx, slot) do { } while (0)
#endif

namespace sdb {

namespace {

constexpr int kTile = 128;         // rows of a query tile and of a key/value block
constexpr int kHeadDim = 128;
#ifndef SDB_FA_THREADS
#define SDB_FA_THREADS 384
#endif
constexpr int kThreads = SDB_FA_THREADS;  // 12 warps: three per scheduler partition of the SM (320: no idle warps)
constexpr int kMmaWarp = 8;
constexpr int kLoadWarp = 9;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS0 = 0, kColS1 = 128, kColO0 = 256, kColO1 = 384;
// ---- build-time choices, each measured at the benchmark shape (B1 N40 S75600, bf16 unless noted) ----------
//
// How the softmax warps treat a block of two-byte operands (e4m3 always takes the block max first):
//   0  exponentials against the running max right away, overflow caught by a row-sum test, P handed over
//      whole; the first block's max, the masking of a partial block and the redo are inline
//   2  block max first; P stored chunk by chunk as it is computed and handed over after 96 and 128
//      keys; the row sum is taken after the hand-over, off the path the MMA thread waits on
//   4  as 0, with everything rare -- the first block's max, the masking (done where the scores lie, in
//      tensor memory), the redo's max and the rescale of O -- in out-of-line functions, so that the loop
//      over the key blocks holds one copy of the exponential pass and nothing else
//   5  as 4, the scores read 32 columns at a time with the next read in flight under the exponentials
// Measured, all builds alternating in one process on one GPU: 0: 102.6 ms, 2: 103.7 ms, 4: 98.3-99.7 ms,
// 5: 98.5-100.4 ms (the earlier kernel: 106.4-107.8 ms).  The code the compiler emits for the loop is
// sensitive to what else is inlined into it: the same pass is 4 % faster with the rare paths out of line, and
// an extra polling loop in front of every barrier wait cost 6 %.
#ifndef SDB_FA_BF16_MODE
#define SDB_FA_BF16_MODE 4
#endif
// Of the eight groups of four scores in a 32-column chunk, how many take the exponentials of their
// second pair on the FMA pipe (ex2_poly2) instead of the exponent unit: 8 = half of all exponentials.
// Measured: the e4m3 kernel, whose softmax loop is bound by the exponent unit, gains with a quarter of its
// exponentials moved (86.5 ms against 92.8 ms) and loses with half; the two-byte kernels, bound by
// instruction issue and latency in that loop, lose with any (a quarter: -2 %, half: -12 %).
#ifndef SDB_FA_POLY
#define SDB_FA_POLY 0
#endif
#ifndef SDB_FA_POLY_FP8
#define SDB_FA_POLY_FP8 4
#endif
// e4m3 sums its probabilities as it goes (1: after the hand-over, like the two-byte max-first form).
#ifndef SDB_FA_DEFER_SUM_FP8
#define SDB_FA_DEFER_SUM_FP8 0
#endif
// Not built: a re-split of the registers between the warpgroups after the roles part (setmaxnreg, 216 for
// the softmax warps and 72 for the others out of the 384 x 168 the launch gives the thread block).  It
// measured the same or slower (104.0-105.0 ms against 103.3-103.9 ms) and does not assemble together
// with out-of-line functions.
constexpr int kBf16Mode = SDB_FA_BF16_MODE;
static_assert(kBf16Mode == 0 || kBf16Mode == 2 || kBf16Mode == 4 || kBf16Mode == 5, "SDB_FA_BF16_MODE");
constexpr bool kLean = kBf16Mode == 4 || kBf16Mode == 5;
constexpr bool kLeanStream = kBf16Mode == 5;
constexpr bool kMaxFirst = kBf16Mode == 2;
constexpr float kRescaleThreshold = 8.0f;  // log2 units the running max may lag before O is rescaled
constexpr float kFp8PShiftLog2 = 8.0f;     // e4m3 probabilities are stored as p * 2^8
constexpr float kFp8Lag = 0.75f;           // 2^8.75 = 431 still fits e4m3 (max 448)

template <bool kFp8>
struct Cfg {
    static constexpr int kElemBytes = kFp8 ? 1 : 2;
    static constexpr int kRowBytes = kHeadDim * kElemBytes;       // 256 / 128
    static constexpr int kAtoms = kRowBytes / 128;                // 128-byte swizzle atoms per row
    static constexpr int kAtomBytes = kTile * 128;                // 16 KB: 128 rows of one atom
    static constexpr int kTileBytes = kAtoms * kAtomBytes;        // 32 KB / 16 KB
    static constexpr int kStages = kFp8 ? 8 : 4;                  // ring slots, each one K or V block
    static constexpr int kBoxInner = 128 / kElemBytes;            // elements of one 128-byte row
    static constexpr int kQkSteps = kRowBytes / 32;               // MMAs per S block (32 B of K-dim each)
    static constexpr int kPvK = 32 / kElemBytes;                  // kv rows per PV MMA (16 / 32)
    static constexpr int kPvSteps = kTile / kPvK;                 // 8 / 4
    static constexpr int kSmemBytes = 2 * kTileBytes + kStages * kTileBytes + 2 * kMaxKvBlocks + 256;
};

struct Ring {
    int idx = 0;
    uint32_t phase = 0;
    template <int N>
    __device__ __forceinline__ void next() {
        if (++idx == N) {
            idx = 0;
            phase ^= 1u;
        }
    }
};

__device__ __forceinline__ uint32_t pack_pair(float lo, float hi, int dtype) {
    if (dtype == 0) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ uint32_t pack_quad_e4m3(float a, float b, float c, float d) {
    uint16_t lo, hi;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
    return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

// Fills one output row (and its log-sum-exp) with NaN: what a thread block leaves behind when it did not
// compute its rows, so that a result produced after a wait gave up can never pass for a real one.
__device__ __forceinline__ void poison_row(const FaParams& p, int batch, int head, int q_row) {
    const int64_t off = batch * p.o_stride[0] + head * p.o_stride[1] + static_cast<int64_t>(q_row) * p.o_stride[2];
    if (p.out_dtype == 2) {
        uint4* dst = reinterpret_cast<uint4*>(static_cast<float*>(p.out) + off);
        const uint4 nan4 = make_uint4(0x7fc00000u, 0x7fc00000u, 0x7fc00000u, 0x7fc00000u);
        for (int i = 0; i < kHeadDim / 4; ++i) dst[i] = nan4;
    } else {
        uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.out) + off);
        const uint32_t n2 = p.out_dtype == 0 ? 0x7fc07fc0u : 0x7e007e00u;
        const uint4 nan4 = make_uint4(n2, n2, n2, n2);
        for (int i = 0; i < kHeadDim / 8; ++i) dst[i] = nan4;
    }
    if (p.lse) p.lse[batch * p.lse_stride[0] + head * p.lse_stride[1] + q_row * p.lse_stride[2]] = __int_as_float(0x7fc00000);
}

// Rare work of a score block, kept out of line so that it costs the hot loop neither registers nor code.
// Fetches the calling row's 128 scores from tensor memory, turns the ones from column n_seen on into
// -inf IN tensor memory (so that every later read sees them masked) and returns the row's maximum.
__device__ __noinline__ float rare_row_max(uint32_t taddr_s, int n_seen) {
    float mx = -INFINITY;
    bool stored = false;
#pragma unroll 1
    for (int c = 0; c < 16; ++c) {
        uint32_t s[8];
        tmem_ld8(taddr_s + c * 8, s);
        tmem_wait_ld();
        // The rows of a warp may see different numbers of columns (causal diagonal); the store is
        // warp-collective, so the warp decides together and a row with nothing to mask writes back what it read.
        if (__any_sync(0xffffffffu, c * 8 + 8 > n_seen)) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (c * 8 + i >= n_seen) s[i] = 0xff800000u;
            tmem_st8(taddr_s + c * 8, s);
            stored = true;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) mx = fmaxf(mx, __uint_as_float(s[i]));
    }
    if (stored) tmem_wait_st();
    return mx;
}

// O *= alpha for the calling row (the accumulator is at rest).
__device__ __noinline__ void rare_rescale_o(uint32_t taddr_o, float alpha) {
#pragma unroll 1
    for (int c = 0; c < kHeadDim / 8; ++c) {
        uint32_t o[8];
        tmem_ld8(taddr_o + c * 8, o);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
        tmem_st8(taddr_o + c * 8, o);
    }
    tmem_wait_st();
}

}  // namespace

// kIn: element type of q/k/v and of the stored probabilities (0 bf16, 1 fp16, 3 e4m3).
// kPairs: the two query tiles of a thread block are the two 128-row blocks a table names (block-sparse
// attention with tiles paired by the similarity of their key lists) instead of two neighbours.
template <int kIn, bool kPairs = false>
__global__ void __launch_bounds__(kThreads, 1) fa_fwd_kernel(const __grid_constant__ FaParams p) {
    constexpr bool kFp8 = kIn == 3;
    constexpr bool kSplit = kFp8 || kMaxFirst;  // P is handed to the MMA thread in two parts
    // 32-key chunks of a block in the first part: half of the block, or three quarters when the
    // exponentials of a two-byte block are taken max-first (the second part's product is then short).
    constexpr int kFirstChunks = (!kFp8 && kMaxFirst) ? 3 : 2;
    using C = Cfg<kFp8>;
    extern __shared__ uint8_t smem_raw[];
    // The swizzle pattern of TMA and of the MMA descriptors is a function of the address bits, so
    // operand tiles start on 1024-byte boundaries.
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sm_q = smem;                              // 2 tiles
    uint8_t* sm_ring = smem + 2 * C::kTileBytes;       // kStages blocks
    uint8_t* sm_flags = sm_ring + C::kStages * C::kTileBytes;  // [2][kMaxKvBlocks]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm_flags + 2 * kMaxKvBlocks);
    // barrier map
    const uint32_t bar_base = smem_u32(bars);
    auto bar_q = [&]() { return bar_base; };
    auto bar_full = [&](int s) { return bar_base + 8u * (1 + s); };
    auto bar_empty = [&](int s) { return bar_base + 8u * (1 + C::kStages + s); };
    auto bar_s = [&](int t) { return bar_base + 8u * (1 + 2 * C::kStages + t); };
    // e4m3: probabilities are handed over in two halves (keys 0-63, 64-127) so that the first half of
    // the P V product runs while the second half of the exponentials is still being taken.  Two-byte
    // operands hand a block over whole, on the second barrier.
    auto bar_p = [&](int t, int h) { return bar_base + 8u * (3 + 2 * C::kStages + 2 * t + h); };
    auto bar_done = [&]() { return bar_base + 8u * (7 + 2 * C::kStages); };
    constexpr int kNumBars = 8 + 2 * C::kStages;
    static_assert(kNumBars * 8 + 16 <= 256, "barrier area");
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* abort_site = abort_flag + 1;  // which wait gave up first (diagnostics)

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int head = blockIdx.y;
    const int batch = blockIdx.z;
    const int kv_head = head / (p.heads / p.kv_heads);
    // The sequence this thread block works on: the whole token axis, or -- packed variable-length
    // sequences -- the one its tile pair falls into.  Rows and keys below are counted from the start of
    // that sequence; q_base / k_base are where it starts on the token axis.
    int qpair = blockIdx.x;
    int q_base = 0, k_base = 0, q_len = p.seq_q, k_len = p.seq_kv;
    if (p.cu_seqlens_q) {
        int i = 0;
        for (; i < p.num_seqs; ++i) {
            const int pairs = (p.cu_seqlens_q[i + 1] - p.cu_seqlens_q[i] + 2 * kTile - 1) / (2 * kTile);
            if (qpair < pairs) break;
            qpair -= pairs;
        }
        if (i == p.num_seqs) return;  // the grid is an upper bound on the number of tile pairs
        q_base = p.cu_seqlens_q[i];
        q_len = p.cu_seqlens_q[i + 1] - q_base;
        k_base = p.cu_seqlens_kv[i];
        k_len = p.cu_seqlens_kv[i + 1] - k_base;
    } else if (p.causal) {
        qpair = static_cast<int>(gridDim.x) - 1 - qpair;  // the tiles with the most visible keys start first
    }
    const int q_row0 = qpair * 2 * kTile;
    // First row of each tile: two neighbouring 128-row blocks, or the two blocks the pairing table names
    // (-1: this thread block has one tile only).
    int pair_blk[2] = {0, 0};
    if constexpr (kPairs) {
        const int32_t* pr = p.q_pairs + ((static_cast<int64_t>(batch) * p.heads + head) * gridDim.x + qpair) * 2;
        pair_blk[0] = pr[0];
        pair_blk[1] = pr[1];
    }
    auto tile_row0 = [&](int t) -> int {
        if constexpr (kPairs) return pair_blk[t] * kTile;
        else return q_row0 + t * kTile;
    };
    const bool tile1_valid = kPairs ? (pair_blk[1] >= 0 && pair_blk[1] * kTile < q_len) : (q_row0 + kTile < q_len);
    // Row of the output that thread tid < 256 answers for when its thread block does not compute (NaN marking).
    auto marked_row = [&](int i) -> int {
        if constexpr (kPairs) return (i < kTile || tile1_valid) ? tile_row0(i >> 7) + (i & (kTile - 1)) : q_len;
        else return q_row0 + i;
    };
    const int nkb = p.cu_seqlens_q ? min((k_len + kTile - 1) / kTile, kMaxKvBlocks) : p.kv_blocks;
    // Causal attention, aligned to the last query and the last key of the sequence: query i sees key j
    // iff j <= i + causal_off.  vis[t]: key blocks tile t can see at all.
    const int causal_off = k_len - q_len;
    int vis[2] = {nkb, nkb};
    if (p.causal) {
        for (int t = 0; t < 2; ++t) {
            const int last_key = tile_row0(t) + kTile - 1 + causal_off;  // of the tile's last row
            vis[t] = last_key < 0 ? 0 : min(nkb, last_key / kTile + 1);
        }
    }

    // A grid in which one CTA already gave up a wait is not going to produce a usable result: the
    // remaining CTAs leave at once instead of each running into its own time-out.
    // The decision is taken once per thread block: all of its threads stay or all leave (the ones that stay
    // set up barriers and tensor memory for the others).  A block that leaves marks its rows.
    if (__syncthreads_or(tid == 0 && p.status && *reinterpret_cast<volatile int*>(p.status) != 0)) {
        if (tid < 2 * kTile && marked_row(tid) < q_len)
            poison_row(p, batch, head, q_base + (p.perm_on ? source_of(make_grid(p.perm_t, p.perm_h, p.perm_w, p.perm_txt), marked_row(tid))
                                                           : marked_row(tid)));
        return;
    }
    const uint32_t wait_us = p.wait_limit_us;

    // ---- set-up -------------------------------------------------------------------------------
    if (tid == 0) {
        mbar_init(bar_q(), 1);
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(bar_full(s), 1);
            mbar_init(bar_empty(s), 1);
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(bar_s(t), 1);
            mbar_init(bar_p(t, 0), kTile);
            mbar_init(bar_p(t, 1), kTile);
        }
        mbar_init(bar_done(), 1);
        *abort_flag = 0;
        *abort_site = 0;
        fence_mbar_init();
    }
    if (warp == kLoadWarp && lane == 0) {
        tma_prefetch_desc(&p.tm_q);
        tma_prefetch_desc(&p.tm_k);
        tma_prefetch_desc(&p.tm_v);
    }
    if (warp == 0) {
        __syncwarp();
        tmem_alloc(smem_u32(tmem_slot), kTmemCols);
        tmem_relinquish();
    }
    // Which kv blocks each tile attends to: one byte per (tile, block).
    {
        uint8_t* f0 = sm_flags;
        uint8_t* f1 = sm_flags + kMaxKvBlocks;
        const int qb0 = qpair * 2;
        auto q_block = [&](int t) -> int {
            if constexpr (kPairs) return pair_blk[t] >= 0 ? pair_blk[t] : pair_blk[0];
            else return qb0 + t;
        };
        if (p.sparse_mode == 0) {
            for (int j = tid; j < nkb; j += kThreads) {
                f0[j] = j < vis[0];
                f1[j] = tile1_valid && j < vis[1];
            }
        } else if (p.sparse_mode == 1) {
            const int8_t* mh = p.block_mask + batch * p.mask_stride[0] + head * p.mask_stride[1];
            const int8_t* m0 = mh + static_cast<int64_t>(q_block(0)) * p.mask_stride[2];
            const int8_t* m1 = mh + static_cast<int64_t>(q_block(1)) * p.mask_stride[2];
            for (int j = tid; j < nkb; j += kThreads) {
                f0[j] = m0[j] != 0 && j < vis[0];
                f1[j] = tile1_valid && m1[j] != 0 && j < vis[1];
            }
        } else {
            for (int j = tid; j < nkb; j += kThreads) {
                f0[j] = 0;
                f1[j] = 0;
            }
            __syncthreads();
            for (int t = 0; t < (tile1_valid ? 2 : 1); ++t) {
                const int64_t row = static_cast<int64_t>(q_block(t)) * p.heads + head;
                const int64_t* ids = p.select_idx + row * p.select_stride;
                int64_t n = p.select_num[row];
                if (n > nkb) n = nkb;
                uint8_t* f = t ? f1 : f0;
                for (int i = tid; i < n; i += kThreads) {
                    const int64_t id = ids[i];
                    if (id >= 0 && id < vis[t]) f[id] = 1;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint8_t* f0 = sm_flags;
    const uint8_t* f1 = sm_flags + kMaxKvBlocks;
    auto flags_of = [&](int j) -> int { return static_cast<int>(f0[j]) | (static_cast<int>(f1[j]) << 1); };
    auto next_block = [&](int j) -> int {
        while (j < nkb && flags_of(j) == 0) ++j;
        return j < nkb ? j : -1;
    };

    if (warp >= 8) {
      if (warp == kLoadWarp && p.perm_on == 1) {
        // ---- TMA producer, RainFusion window permutation applied on the fly ---------------------
        // q, k and v are in their original token order; the tiles the other roles see hold the PERMUTED
        // order.  Eight consecutive positions of the permuted order are eight consecutive source tokens
        // (the launcher checked that the grid allows it), so a 128-row tile is 16 copies of 8 tokens per
        // 64-channel atom: each lane of the warp owns one (group, atom) and issues one 1 KB copy per tile.
        if constexpr (!kFp8) {
            const Grid grid = make_grid(p.perm_t, p.perm_h, p.perm_w, p.perm_txt);
            const int grp = lane & 15, atom = lane >> 4;
            // first source token of the eight-row group at position pos; past the end: out of range, which
            // the copy engine fills with zeros
            auto group_token = [&](int pos, int len) { return pos < len ? source_of(grid, pos) : len; };
            const uint32_t my_off = static_cast<uint32_t>(atom * C::kAtomBytes + grp * 1024);
            if (lane == 0) mbar_arrive_expect_tx(bar_q(), (tile1_valid ? 2 : 1) * C::kTileBytes);
            __syncwarp();
            for (int t = 0; t < (tile1_valid ? 2 : 1); ++t)
                tma_load_4d(smem_u32(sm_q + t * C::kTileBytes) + my_off, &p.tm_q8, bar_q(), atom * C::kBoxInner,
                            group_token(tile_row0(t) + grp * 8, q_len), head, batch);
            Ring ring;
            int issued = 0;
            bool ok = true;
            for (int u = next_block(0); u >= 0 && ok; u = next_block(u + 1)) {
                const int tok = group_token(u * kTile + grp * 8, k_len);
                for (int which = 0; which < 2 && ok; ++which) {  // 0: K block, 1: V block
                    ok = __all_sync(0xffffffffu, mbar_wait(bar_empty(ring.idx), ring.phase ^ 1u, abort_flag, 1, wait_us));
                    if (!ok) break;
                    if (lane == 0) mbar_arrive_expect_tx(bar_full(ring.idx), C::kTileBytes);
                    __syncwarp();
                    tma_load_4d(smem_u32(sm_ring + ring.idx * C::kTileBytes) + my_off, which ? &p.tm_v8 : &p.tm_k8,
                                bar_full(ring.idx), atom * C::kBoxInner, tok, kv_head, batch);
                    ring.template next<C::kStages>();
                    ++issued;
                }
            }
            // Before the CTA may exit, every copy this warp started must have landed.
            mbar_wait_drain(bar_q(), 0);
            const int pending = issued < C::kStages ? issued : C::kStages;
            for (int i = 0; i < pending; ++i) {
                const int n = issued - 1 - i;
                mbar_wait_drain(bar_full(n % C::kStages), static_cast<uint32_t>(n / C::kStages) & 1u);
            }
        }
      } else if (warp == kLoadWarp) {
        // ---- TMA producer ---------------------------------------------------------------------
        if (lane == 0) {
            const uint32_t q_bytes = (tile1_valid ? 2 : 1) * C::kTileBytes;
            mbar_arrive_expect_tx(bar_q(), q_bytes);
            for (int t = 0; t < (tile1_valid ? 2 : 1); ++t)
                for (int a = 0; a < C::kAtoms; ++a)
                    tma_load_4d(smem_u32(sm_q + t * C::kTileBytes + a * C::kAtomBytes), &p.tm_q, bar_q(),
                                a * C::kBoxInner, q_base + tile_row0(t), head, batch);
            Ring ring;
            int issued = 0, withheld = -1;
            bool ok = true;
            for (int u = next_block(0); u >= 0 && ok; u = next_block(u + 1)) {
                for (int which = 0; which < 2 && ok; ++which) {  // 0: K block, 1: V block
                    ok = mbar_wait(bar_empty(ring.idx), ring.phase ^ 1u, abort_flag, 1, wait_us);
                    if (!ok) break;
                    if (p.test_withhold && issued == 0) {
                        // Host-side failure injection for the tests of the bounded waits: the first copy is
                        // neither started nor announced, so its barrier never completes, the consumer's wait
                        // runs into the limit and the thread block unwinds.  Nothing is in flight for it.
                        withheld = 0;
                    } else {
                        mbar_arrive_expect_tx(bar_full(ring.idx), C::kTileBytes);
                        const CUtensorMap* tm = which ? &p.tm_v : &p.tm_k;
                        for (int a = 0; a < C::kAtoms; ++a)
                            tma_load_4d(smem_u32(sm_ring + ring.idx * C::kTileBytes + a * C::kAtomBytes), tm,
                                        bar_full(ring.idx), a * C::kBoxInner, k_base + u * kTile, kv_head, batch);
                    }
                    ring.template next<C::kStages>();
                    ++issued;
                }
            }
            // Before the CTA may exit, every copy this thread started must have landed.
            mbar_wait_drain(bar_q(), 0);
            const int pending = issued < C::kStages ? issued : C::kStages;
            for (int i = 0; i < pending; ++i) {
                const int n = issued - 1 - i;  // n-th load overall
                if (n == withheld) continue;   // never started
                mbar_wait_drain(bar_full(n % C::kStages), static_cast<uint32_t>(n / C::kStages) & 1u);
            }
        }
    } else if (warp == kMmaWarp) {
        // ---- MMA issue ------------------------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t fmt = kIn == 0 ? 1u : 0u;  // f16 kind: 1 = bf16, 0 = fp16; f8f6f4 kind: 0 = e4m3
            const uint32_t idesc_qk = umma_idesc(fmt, kTile, kTile, false, false);
            const uint32_t idesc_pv = umma_idesc(fmt, kTile, kHeadDim, false, true);
            const uint32_t col_s[2] = {tmem_base + kColS0, tmem_base + kColS1};
            const uint32_t col_o[2] = {tmem_base + kColO0, tmem_base + kColO1};

            const uint32_t q_lo[2] = {desc_lo(smem_u32(sm_q), 16), desc_lo(smem_u32(sm_q + C::kTileBytes), 16)};
            const uint32_t ring_k_lo = desc_lo(smem_u32(sm_ring), 16);
            const uint32_t ring_v_lo = desc_lo(smem_u32(sm_ring), C::kAtomBytes);
            constexpr uint32_t kSlotStep = C::kTileBytes >> 4;
            auto issue_s = [&](int t, int slot) {
                const uint32_t k_lo = ring_k_lo + slot * kSlotStep;
#pragma unroll
                for (int kc = 0; kc < C::kQkSteps; ++kc) {
                    constexpr uint32_t kAtom16 = C::kAtomBytes >> 4;
                    const uint32_t off = (kc >> 2) * kAtom16 + (kc & 3) * 2;
                    umma_ss_lohi<kFp8>(col_s[t], q_lo[t] + off, k_lo + off, kDescHiSbo1024, idesc_qk, kc > 0);
                }
                umma_commit(bar_s(t));
            };
            constexpr int kFirstSteps = C::kPvSteps * kFirstChunks / 4;
            auto issue_pv = [&](int t, int h, int slot, bool accumulate) {  // first (h = 0) or second part of the block's keys
                const uint32_t v_lo = ring_v_lo + slot * kSlotStep;
#pragma unroll
                for (int kc = 0; kc < C::kPvSteps; ++kc) {
                    if ((kc < kFirstSteps) != (h == 0)) continue;
                    umma_ts_lohi<kFp8>(col_o[t], col_s[t] + kc * 8, v_lo + kc * (C::kPvK * 128 >> 4), kDescHiSbo1024, idesc_pv,
                                       (accumulate || kc > 0) ? 1u : 0u);
                }
            };

            bool ok = mbar_wait(bar_q(), 0, abort_flag, 10, wait_us);
            Ring ring;
            int pv_cnt[2] = {0, 0};
            int u = next_block(0);
            if (ok && u >= 0) {
                ok = mbar_wait(bar_full(ring.idx), ring.phase, abort_flag, 11, wait_us);
                if (ok) {
                    tc_fence_after();
                    const int f = flags_of(u);
                    if (f & 1) issue_s(0, ring.idx);
                    if (f & 2) issue_s(1, ring.idx);
                    umma_commit(bar_empty(ring.idx));
                    ring.template next<C::kStages>();
                }
            }
            while (ok && u >= 0) {
                const int f = flags_of(u);
                const int nu = next_block(u + 1);
                const int nf = nu >= 0 ? flags_of(nu) : 0;
                const Ring vslot = ring;
                ring.template next<C::kStages>();
                const Ring kslot = ring;
                if (nf) ring.template next<C::kStages>();

                ok = mbar_wait(bar_full(vslot.idx), vslot.phase, abort_flag, 12, wait_us);
                if (!ok) break;
                SDB_TR(2, u, 0);
                if (f & 1) {
                    if constexpr (kSplit) {
                        ok = mbar_wait(bar_p(0, 0), static_cast<uint32_t>(pv_cnt[0]) & 1u, abort_flag, 13, wait_us);
                        if (!ok) break;
                        tc_fence_after();
                        SDB_TR(2, u, 1);
                        issue_pv(0, 0, vslot.idx, pv_cnt[0] > 0);
                        SDB_TR(2, u, 2);
                    }
                    ok = mbar_wait(bar_p(0, 1), static_cast<uint32_t>(pv_cnt[0]) & 1u, abort_flag, 13, wait_us);
                    if (!ok) break;
                    tc_fence_after();
                    SDB_TR(2, u, 3);
                    if constexpr (!kSplit) issue_pv(0, 0, vslot.idx, pv_cnt[0] > 0);
                    issue_pv(0, 1, vslot.idx, true);
                    ++pv_cnt[0];
                    SDB_TR(2, u, 4);
                }
                if (nf) {
                    ok = mbar_wait(bar_full(kslot.idx), kslot.phase, abort_flag, 17, wait_us);
                    if (!ok) break;
                    tc_fence_after();
                }
                if (nf & 1) issue_s(0, kslot.idx);
                SDB_TR(2, u, 5);
                if (f & 2) {
                    if constexpr (kSplit) {
                        ok = mbar_wait(bar_p(1, 0), static_cast<uint32_t>(pv_cnt[1]) & 1u, abort_flag, 14, wait_us);
                        if (!ok) break;
                        tc_fence_after();
                        SDB_TR(2, u, 6);
                        issue_pv(1, 0, vslot.idx, pv_cnt[1] > 0);
                        SDB_TR(2, u, 7);
                    }
                    ok = mbar_wait(bar_p(1, 1), static_cast<uint32_t>(pv_cnt[1]) & 1u, abort_flag, 14, wait_us);
                    if (!ok) break;
                    tc_fence_after();
                    SDB_TR(2, u, 8);
                    if constexpr (!kSplit) issue_pv(1, 0, vslot.idx, pv_cnt[1] > 0);
                    issue_pv(1, 1, vslot.idx, true);
                    ++pv_cnt[1];
                    SDB_TR(2, u, 9);
                }
                umma_commit(bar_empty(vslot.idx));
                if (nf & 2) issue_s(1, kslot.idx);
                SDB_TR(2, u, 10);
                if (nf) umma_commit(bar_empty(kslot.idx));
                u = nu;
            }
            // Final arrival on each tile's S barrier: its output accumulator is complete.
            umma_commit(bar_s(0));
            umma_commit(bar_s(1));
            if (!ok) {
                // Unwinding: tensor memory is about to be freed, so the products already issued must be over.
                umma_commit(bar_done());
                mbar_wait_drain(bar_done(), 0);
            }
        }
      }
    } else {
        // ---- softmax, O rescale, epilogue: one query row per thread ------------------------------
        const int t = warp >> 2;  // tile of this warpgroup
        const int row_in_tile = tid & (kTile - 1);
        const int q_row = tile_row0(t) + row_in_tile;
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t taddr_s = tmem_base + (t ? kColS1 : kColS0) + lane_base;
        const uint32_t taddr_o = tmem_base + (t ? kColO1 : kColO0) + lane_base;
        const uint8_t* my_flags = t ? f1 : f0;
        const int tail_valid = k_len - (nkb - 1) * kTile;  // valid columns of the last kv block
        const int tile_last_key = tile_row0(t) + causal_off;  // last key the tile's FIRST row sees
        // The running max may lag the true max by this much (log2 units) before O is rescaled; the
        // probabilities then reach 2^lag, which two-byte formats hold but e4m3 does not.
        constexpr float kLag = kFp8 ? kFp8Lag : kRescaleThreshold;
        constexpr float kRedoSum = 256.0f;  // 2^kRescaleThreshold

        // e4m3: the dequantisation scales of the q block and of each k block fold into the
        // exponent's multiplier; a per-token-block v scale folds into the exponent's offset.
        float q_sc = 1.0f, v_ref = 1.0f;
        const float* k_sc = nullptr;
        const float* v_blk = nullptr;
        if constexpr (kFp8) {
            int qb = tile_row0(t) / kTile;
            if (qb >= p.q_blocks) qb = p.q_blocks - 1;
            q_sc = p.q_scale[(static_cast<int64_t>(batch) * p.heads + head) * p.q_blocks + qb];
            k_sc = p.k_scale + (static_cast<int64_t>(batch) * p.kv_heads + kv_head) * p.k_scale_count;
            if (p.v_scale_block > 0) {
                v_blk = p.v_scale + (static_cast<int64_t>(batch) * p.kv_heads + kv_head) * p.v_scale_count;
                float mx = 0.0f;
                for (int i = lane; i < p.v_scale_count; i += 32) mx = fmaxf(mx, v_blk[i]);
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
                v_ref = mx > 0.0f ? mx : 1.0f;
            }
        }

        // scale blocks are 128, 256 or 512 tokens: key block j uses scale j >> shift
        int k_shift = 0, v_shift = 0;
        if constexpr (kFp8) {
            k_shift = 31 - __clz(p.k_scale_block / kTile);
            if (p.v_scale_block > 0) v_shift = 31 - __clz(p.v_scale_block / kTile);
        }
        float m_run = -INFINITY;  // running row max, in log2 units of the scaled scores
        float l_run = 0.0f;
        int cnt = 0;
        bool ok = true;
        for (int j = 0; j < nkb; ++j) {
            if (!my_flags[j]) continue;
            // The block's dequantisation scales are fetched (and the v scale's logarithm taken) before the wait
            // for its scores: their latency is spent while the MMA thread still works on the block.
            float mult = p.scale_log2;
            float v_off = 0.0f, l_fix = 1.0f;
            if constexpr (kFp8) {
                mult *= q_sc * k_sc[j >> k_shift];
                if (v_blk) {
                    const float r = fmaxf(v_blk[j >> v_shift], 1e-30f) / v_ref;
                    v_off = log2f(r);
                    l_fix = 1.0f / r;
                }
            }
            ok = __all_sync(0xffffffffu, mbar_wait(bar_s(t), static_cast<uint32_t>(cnt) & 1u, abort_flag, 20 + t, wait_us));
            if (!ok) break;
            tc_fence_after();
            if (row_in_tile == 64) SDB_TR(t, j, 0);

            // Columns this row may not see in this block: beyond the end of the keys (last block) or, with
            // causal attention, beyond the row's own position (the blocks the tile's diagonal crosses).
            bool masked = j == nkb - 1 && tail_valid < kTile;  // warp-uniform
            int n_seen = masked ? tail_valid : kTile;
            if (p.causal && j * kTile + kTile - 1 > tile_last_key) {
                masked = true;
                n_seen = min(n_seen, q_row + causal_off - j * kTile + 1);
            }
            uint32_t s[4][32];
            constexpr bool kWholeRowFirst = kFp8 || !kLean;  // the lean forms fetch the scores inside their pass loop
            if constexpr (kWholeRowFirst) {
                if constexpr (kFp8)
                    if (masked) rare_row_max(taddr_s, n_seen);  // masks the scores where they lie
#pragma unroll
                for (int c = 0; c < 4; ++c) tmem_ld32(taddr_s + c * 32, s[c]);
                tmem_wait_ld();
            }
            if (row_in_tile == 64) SDB_TR(t, j, 1);
            auto mask_scores = [&]() {
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (c * 32 + i >= n_seen) s[c][i] = 0xff800000u;  // -inf
            };
            if constexpr (kWholeRowFirst && !kFp8)
                if (masked) mask_scores();
            // The four exponentials of one group: x = s * mult - m as packed pairs, the first pair on the
            // exponent unit, the second there too or -- for kPoly of every eight groups -- on the FMA pipe.
            constexpr int kPoly = kFp8 ? SDB_FA_POLY_FP8 : SDB_FA_POLY;
            auto exp4 = [&](auto clamp_high, int c, int i, uint64_t mult2, uint64_t negm2, float& e0, float& e1, float& e2,
                            float& e3) {
                unpack2(fma2(pack2(__uint_as_float(s[c][4 * i]), __uint_as_float(s[c][4 * i + 1])), mult2, negm2), e0, e1);
                e0 = ex2_approx(e0);
                e1 = ex2_approx(e1);
                const uint64_t x23 = fma2(pack2(__uint_as_float(s[c][4 * i + 2]), __uint_as_float(s[c][4 * i + 3])), mult2, negm2);
                if (((i + 1) * kPoly) / 8 > (i * kPoly) / 8) {  // resolved at compile time: i is an unrolled index
                    ex2_poly2<decltype(clamp_high)::value>(x23, e2, e3);
                } else {
                    unpack2(x23, e2, e3);
                    e2 = ex2_approx(e2);
                    e3 = ex2_approx(e3);
                }
            };
            auto row_max = [&]() {
                // Eight independent chains of three-input max: a single running max would be 128 dependent
                // instructions.
                float mx8[8];
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    mx8[i] = fmax3(__uint_as_float(s[0][i]), __uint_as_float(s[0][i + 8]), __uint_as_float(s[0][i + 16]));
#pragma unroll
                for (int i = 0; i < 8; ++i) mx8[i] = fmax3(mx8[i], __uint_as_float(s[0][i + 24]), __uint_as_float(s[1][i]));
#pragma unroll
                for (int i = 0; i < 8; ++i) mx8[i] = fmax3(mx8[i], __uint_as_float(s[1][i + 8]), __uint_as_float(s[1][i + 16]));
#pragma unroll
                for (int i = 0; i < 8; ++i) mx8[i] = fmax3(mx8[i], __uint_as_float(s[1][i + 24]), __uint_as_float(s[2][i]));
#pragma unroll
                for (int i = 0; i < 8; ++i) mx8[i] = fmax3(mx8[i], __uint_as_float(s[2][i + 8]), __uint_as_float(s[2][i + 16]));
#pragma unroll
                for (int i = 0; i < 8; ++i) mx8[i] = fmax3(mx8[i], __uint_as_float(s[2][i + 24]), __uint_as_float(s[3][i]));
#pragma unroll
                for (int i = 0; i < 8; ++i) mx8[i] = fmax3(mx8[i], __uint_as_float(s[3][i + 8]), __uint_as_float(s[3][i + 16]));
#pragma unroll
                for (int i = 0; i < 8; ++i) mx8[i] = fmaxf(mx8[i], __uint_as_float(s[3][i + 24]));
                return fmaxf(fmax3(mx8[0], mx8[1], mx8[2]), fmaxf(fmax3(mx8[3], mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
            };
            if constexpr (!kFp8 && kLean) {
                // As the next form, with everything that is rare -- the first block's max, masking, the redo --
                // in out-of-line functions that work on tensor memory.
                const bool first = cnt == 0;
                if (masked || first) {
                    const float mx = rare_row_max(taddr_s, masked ? n_seen : kTile);
                    if (first) m_run = fmaxf(mx * mult, -3.0e38f);
                }
                const uint64_t mult2 = pack2(mult, mult);
                uint32_t pk[4][16];
                float sum = 0.0f;
    #pragma unroll 1
                for (int pass = 0; pass < 2; ++pass) {
                    const float neg_m = -m_run;
                    const uint64_t negm2 = pack2(neg_m, neg_m);
                    uint64_t sum2[2] = {pack2(0.0f, 0.0f), pack2(0.0f, 0.0f)};
                    if constexpr (kLeanStream) {
                        // 32 columns at a time, the next read in flight under the exponentials of the previous ones
                        tmem_ld32(taddr_s, s[0]);
    #pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            tmem_wait_ld();
                            if (c < 3) tmem_ld32(taddr_s + (c + 1) * 32, s[(c + 1) & 1]);
    #pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                float e0, e1, e2, e3;
                                exp4(std::true_type{}, c & 1, i, mult2, negm2, e0, e1, e2, e3);
                                sum2[0] = add2(sum2[0], pack2(e0, e1));
                                sum2[1] = add2(sum2[1], pack2(e2, e3));
                                pk[c][2 * i] = pack_pair(e0, e1, kIn);
                                pk[c][2 * i + 1] = pack_pair(e2, e3, kIn);
                            }
                        }
                    } else {
    #pragma unroll
                        for (int c = 0; c < 4; ++c) tmem_ld32(taddr_s + c * 32, s[c]);
                        tmem_wait_ld();
    #pragma unroll
                        for (int c = 0; c < 4; ++c) {
    #pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                float e0, e1, e2, e3;
                                exp4(std::true_type{}, c, i, mult2, negm2, e0, e1, e2, e3);
                                sum2[0] = add2(sum2[0], pack2(e0, e1));
                                sum2[1] = add2(sum2[1], pack2(e2, e3));
                                pk[c][2 * i] = pack_pair(e0, e1, kIn);
                                pk[c][2 * i + 1] = pack_pair(e2, e3, kIn);
                            }
                        }
                    }
                    {
                        float a, b;
                        unpack2(add2(sum2[0], sum2[1]), a, b);
                        sum = a + b;
                    }
                    if (pass == 1 || first) break;
                    if (!__any_sync(0xffffffffu, !(sum <= kRedoSum))) break;
                    const float m_new = fmaxf(m_run, rare_row_max(taddr_s, kTile) * mult);
                    const float alpha = ex2_approx(m_run - m_new);
                    m_run = m_new;
                    l_run *= alpha;
                    rare_rescale_o(taddr_o, alpha);
                }
    #pragma unroll
                for (int c = 0; c < 4; ++c) tmem_st16(taddr_s + c * 16, pk[c]);
                l_run += sum;
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(bar_p(t, 1));
            } else if constexpr (!kFp8 && !kMaxFirst) {
                // The probabilities are taken against the running max right away and kept in registers; the
                // scores die as they are consumed.  Every probability is non-negative, so a row sum within
                // 2^lag bounds each of them: only if that test fails somewhere in the warp -- rare after the
                // first blocks -- are the scores fetched again (nothing has been stored over them yet), the
                // block's own max taken, O and the running sum rescaled, and the probabilities redone.  The
                // first block has no running max yet and takes its own first.
                // A row that sees no key of its first block sees none at all (causal): any finite max
                // gives it zero probabilities and a zero sum.
                if (cnt == 0) m_run = fmaxf(row_max() * mult, -3.0e38f);
                const uint64_t mult2 = pack2(mult, mult);
                uint32_t pk[4][16];
                float sum = 0.0f;
    #pragma unroll 1
                for (int pass = 0; pass < 2; ++pass) {
                    const float neg_m = -m_run;
                    const uint64_t negm2 = pack2(neg_m, neg_m);
                    uint64_t sum2[2] = {pack2(0.0f, 0.0f), pack2(0.0f, 0.0f)};
    #pragma unroll
                    for (int c = 0; c < 4; ++c) {
    #pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            float e0, e1, e2, e3;
                            exp4(std::true_type{}, c, i, mult2, negm2, e0, e1, e2, e3);  // speculative: x has no upper bound
                            sum2[0] = add2(sum2[0], pack2(e0, e1));
                            sum2[1] = add2(sum2[1], pack2(e2, e3));
                            pk[c][2 * i] = pack_pair(e0, e1, kIn);
                            pk[c][2 * i + 1] = pack_pair(e2, e3, kIn);
                        }
                    }
                    {
                        float a, b;
                        unpack2(add2(sum2[0], sum2[1]), a, b);
                        sum = a + b;
                    }
                    if (pass == 1 || cnt == 0) break;
                    if (!__any_sync(0xffffffffu, !(sum <= kRedoSum))) break;
    #pragma unroll
                    for (int c = 0; c < 4; ++c) tmem_ld32(taddr_s + c * 32, s[c]);
                    tmem_wait_ld();
                    if (masked) mask_scores();
                    const float m_new = fmaxf(m_run, row_max() * mult);
                    const float alpha = ex2_approx(m_run - m_new);
                    m_run = m_new;
                    l_run *= alpha;
                    // The previous P V product has finished (the scores were issued behind it) and this
                    // block's has not been handed over: O is at rest.
    #pragma unroll 1
                    for (int c = 0; c < kHeadDim / 8; ++c) {
                        uint32_t o[8];
                        tmem_ld8(taddr_o + c * 8, o);
                        tmem_wait_ld();
    #pragma unroll
                        for (int i = 0; i < 8; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st8(taddr_o + c * 8, o);
                    }
                }
    #pragma unroll
                for (int c = 0; c < 4; ++c) tmem_st16(taddr_s + c * 16, pk[c]);
                l_run += sum;
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(bar_p(t, 1));
            } else {
                // e4m3 leaves less than one binade of lag, so a speculative pass would be redone too often:
                // the block max is taken first.  In exchange the probabilities are handed over in two
                // halves, so the first half of the P V product runs under the second half of the
                // exponentials (the fp8 products are short; their latency matters more than for bf16).
                const float m_cand = row_max() * mult;
                const bool rescale = __any_sync(0xffffffffu, m_cand > m_run + kLag);
                float alpha = 1.0f;
                if (rescale) {
                    const float m_new = fmaxf(m_run, m_cand);
                    alpha = m_new == -INFINITY ? 0.0f : ex2_approx(m_run - m_new);  // 0 on the first block (m_run = -inf)
                    l_run *= alpha;
                    m_run = m_new;
                    // The (rare, after the first blocks) rescale of O must be over before the first half
                    // of P is handed to the MMA thread.  The scores of this block were issued behind the
                    // previous P V product, so that product has finished.
                    if (cnt > 0) rare_rescale_o(taddr_o, alpha);
                }
                if (row_in_tile == 64) SDB_TR(t, j, 2);
                // x = s * mult - m as packed pairs (one instruction per two scores), then ex2 and pack.
                const float neg_m = m_run == -INFINITY ? 0.0f : (kFp8 ? (kFp8PShiftLog2 + v_off - m_run) : -m_run);
                const uint64_t mult2 = pack2(mult, mult), negm2 = pack2(neg_m, neg_m);
                // Two-byte operands take the row sum after the hand-over (the exponentials stay in the
                // scores' registers until then); e4m3 -- whose loop is bound by the exponent unit, with
                // issue slots to spare -- sums as it goes, which keeps fewer values alive.
                constexpr bool kDeferSum = SDB_FA_DEFER_SUM_FP8 || !kFp8;
                uint64_t run2[2] = {pack2(0.0f, 0.0f), pack2(0.0f, 0.0f)};
    #pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t pk[kFp8 ? 8 : 16];
    #pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        float e0, e1, e2, e3;
                        exp4(std::false_type{}, c, i, mult2, negm2, e0, e1, e2, e3);  // x <= the lag: the max was taken first
                        if constexpr (kDeferSum) {
                            s[c][4 * i] = __float_as_uint(e0);
                            s[c][4 * i + 1] = __float_as_uint(e1);
                            s[c][4 * i + 2] = __float_as_uint(e2);
                            s[c][4 * i + 3] = __float_as_uint(e3);
                        } else {
                            run2[0] = add2(run2[0], pack2(e0, e1));
                            run2[1] = add2(run2[1], pack2(e2, e3));
                        }
                        if constexpr (kFp8) {
                            pk[i] = pack_quad_e4m3(e0, e1, e2, e3);
                        } else {
                            pk[2 * i] = pack_pair(e0, e1, kIn);
                            pk[2 * i + 1] = pack_pair(e2, e3, kIn);
                        }
                    }
                    // The packed chunk lands on columns whose scores are already in registers.
                    if constexpr (kFp8) tmem_st8(taddr_s + c * 8, pk);
                    else tmem_st16(taddr_s + c * 16, pk);
                    if (row_in_tile == 64) SDB_TR(t, j, 3 + c);
                    if (c == kFirstChunks - 1 || c == 3) {  // a part of the block's keys is complete: hand it over
                        tmem_wait_st();
                        tc_fence_before();
                        mbar_arrive(bar_p(t, c == 3 ? 1 : 0));
                        if (row_in_tile == 64) SDB_TR(t, j, c == 3 ? 8 : 7);
                    }
                }
                if constexpr (!kDeferSum) {
                    float a, b;
                    unpack2(add2(run2[0], run2[1]), a, b);
                    l_run += (a + b) * l_fix;
                } else {
                    // The row sum, while the MMA thread is busy with what it was just handed.
                    uint64_t sum2[4] = {pack2(0.0f, 0.0f), pack2(0.0f, 0.0f), pack2(0.0f, 0.0f), pack2(0.0f, 0.0f)};
    #pragma unroll
                    for (int c = 0; c < 4; ++c)
    #pragma unroll
                        for (int i = 0; i < 16; ++i)
                            sum2[i & 3] = add2(sum2[i & 3], pack2(__uint_as_float(s[c][2 * i]), __uint_as_float(s[c][2 * i + 1])));
                    float a, b;
                    unpack2(add2(add2(sum2[0], sum2[1]), add2(sum2[2], sum2[3])), a, b);
                    l_run += (a + b) * l_fix;
                }
                if (row_in_tile == 64) SDB_TR(t, j, 9);
            }
            ++cnt;
        }
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar_s(t), static_cast<uint32_t>(cnt) & 1u, abort_flag, 26 + t, wait_us));
        if (ok && (t == 0 || tile1_valid)) {  // warp-uniform: the tensor-memory loads are warp-collective
            tc_fence_after();
            const bool row_ok = q_row < q_len;
            // Row of the output this thread writes: its own position, or -- window permutation on the fly --
            // the source token that position holds, so that the output is in the original order.
            int out_row = q_row;
            if (p.perm_on && row_ok) out_row = source_of(make_grid(p.perm_t, p.perm_h, p.perm_w, p.perm_txt), q_row);
            // l_run carries the 2^8 shift of the stored e4m3 probabilities, so it cancels in O / l.
            // A row that sees no key at all (causal, more queries than keys) gives zeros whatever its
            // masked scores were turned into.
            const bool sees_keys = !p.causal || q_row + causal_off >= 0;
            if (!sees_keys) l_run = 0.0f;
            const float inv_l = l_run > 0.0f ? v_ref / l_run : 0.0f;
            const float* v_ch = (kFp8 && p.v_scale_block == 0)
                                    ? p.v_scale + (static_cast<int64_t>(batch) * p.kv_heads + kv_head) * kHeadDim
                                    : nullptr;
            uint8_t* orow = static_cast<uint8_t*>(p.out) +
                            (batch * p.o_stride[0] + head * p.o_stride[1] + static_cast<int64_t>(q_base + out_row) * p.o_stride[2]) *
                                (p.out_dtype == 2 ? 4 : 2);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t o[32];
                if (cnt > 0) {
                    tmem_ld32(taddr_o + c * 32, o);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = 0;
                }
                float vals[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    float x = __uint_as_float(o[i]) * inv_l;
                    if constexpr (kFp8)
                        if (v_ch) x *= v_ch[c * 32 + i];
                    vals[i] = x;
                }
                if (row_ok) {
                    if (p.out_dtype == 2) {
                        float4* dst = reinterpret_cast<float4*>(orow + c * 128);
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            dst[i] = make_float4(vals[4 * i], vals[4 * i + 1], vals[4 * i + 2], vals[4 * i + 3]);
                    } else {
                        uint4* dst = reinterpret_cast<uint4*>(orow + c * 64);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            uint4 w;
                            w.x = pack_pair(vals[8 * i + 0], vals[8 * i + 1], p.out_dtype);
                            w.y = pack_pair(vals[8 * i + 2], vals[8 * i + 3], p.out_dtype);
                            w.z = pack_pair(vals[8 * i + 4], vals[8 * i + 5], p.out_dtype);
                            w.w = pack_pair(vals[8 * i + 6], vals[8 * i + 7], p.out_dtype);
                            dst[i] = w;
                        }
                    }
                }
            }
#ifndef SDB_FA_TRACE
            if (p.lse && row_ok) {
                const float shift = kFp8 ? kFp8PShiftLog2 : 0.0f;
                p.lse[batch * p.lse_stride[0] + head * p.lse_stride[1] + (q_base + out_row) * p.lse_stride[2]] =
                    l_run > 0.0f ? (m_run - shift) * 0.6931471805599453f + logf(l_run) : -INFINITY;
            }
#endif
        }
    }

    // ---- teardown ---------------------------------------------------------------------------------
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
    if (*abort_flag && tid < 2 * kTile && marked_row(tid) < q_len)
        poison_row(p, batch, head, q_base + (p.perm_on ? source_of(make_grid(p.perm_t, p.perm_h, p.perm_w, p.perm_txt), marked_row(tid))
                                                       : marked_row(tid)));
    if (tid == 0 && *abort_flag && p.status) {
        // First CTA to report wins the word and leaves where it stopped behind it.
        if (atomicCAS(p.status, 0, kStatusFaWaitGaveUp) == 0) {
            p.status[1] = *abort_site;
            p.status[2] = static_cast<int>(blockIdx.x);
            p.status[3] = static_cast<int>(blockIdx.y);
            p.status[4] = static_cast<int>(blockIdx.z);
        }
    }
}

int fa_fwd_smem_bytes(bool fp8) { return (fp8 ? Cfg<true>::kSmemBytes : Cfg<false>::kSmemBytes) + 1024; }

template <int kIn, bool kPairs = false>
static cudaError_t launch_one(const FaParams& p, cudaStream_t stream) {
    const int smem = fa_fwd_smem_bytes(kIn == 3);
    cudaError_t e = cudaFuncSetAttribute(fa_fwd_kernel<kIn, kPairs>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    // Packed sequences: every sequence rounds its tile pairs up, so seq_q / 256 + num_seqs bounds their number.
    const int pairs = kPairs ? p.q_pair_count
                             : (p.cu_seqlens_q ? p.seq_q / (2 * kTile) + p.num_seqs : (p.seq_q + 2 * kTile - 1) / (2 * kTile));
    dim3 grid(pairs, p.heads, p.batch);
    fa_fwd_kernel<kIn, kPairs><<<grid, kThreads, smem, stream>>>(p);
    return cudaGetLastError();
}

cudaError_t fa_fwd_launch(const FaParams& p, cudaStream_t stream) {
    if (p.q_pairs) {  // the caller checked: block mask or lists, two-byte operands, no causal mask, no packed sequences
        if (p.in_dtype == 0) return launch_one<0, true>(p, stream);
        if (p.in_dtype == 1) return launch_one<1, true>(p, stream);
        return cudaErrorInvalidValue;
    }
    switch (p.in_dtype) {
        case 0: return launch_one<0>(p, stream);
        case 1: return launch_one<1>(p, stream);
        case 3: return launch_one<3>(p, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace sdb

// Sparse block estimate (the mask builder of adaptive block-sparse attention) for sm_100a.
//
// What is computed.  Tokens are taken eight at a time ("groups").  The pooled logit of query group
// g and key group h is  s[g, h] = scale * sum_i q[8g + 7 - i] . k[8h + i]  -- one 1024-long dot
// product (8 tokens x 128 channels) along the anti-diagonal of the 8x8 token cell.  Each row of s
// is put through a softmax over all key groups; the probabilities are summed over the 16 key groups
// of a 128-token key block and over the 16 query groups of a 128-token query block.  Per query
// block the heaviest key blocks are then kept until they hold `threshold` of the row's mass.
//
// Kernel 1 (sbe_partial_kernel): the logits are a GEMM with K = 1024 over strided views of q and k,
// so it runs on tcgen05: one CTA owns 128 query groups (M) of one head and walks the key groups 256
// at a time (N), the contraction streamed through a 4-stage TMA ring in 64-channel slices.  Two
// 256-column accumulators in tensor memory alternate, so the exponentials of one trip run under the
// MMAs of the next.  The softmax is single pass: every trip is normalised with the running row
// maximum known at that time, the 16 block sums of the trip are written out per row together with
// that maximum, and the correction to the final maximum is applied by kernel 2.
//   warps 0-3  softmax (one query group per thread)   warp 4  MMA issue   warp 5  TMA loads
//
// Kernel 2 (sbe_select_kernel): one CTA per (query block, head): rescales and normalises the 16
// rows, adds them, finds the guard score of the cumulative-mass rule by a bitwise search (no sort)
// and writes the int8 mask row and the kept count.
#include "capi_common.h"
#include "fa_fwd.h"
#include "ptx_sm100.cuh"

#include <cmath>

namespace sdb {

namespace {

constexpr int kGroup = 8;          // tokens per group (the operator's `stride`)
constexpr int kRows = 128;         // query groups per CTA
constexpr int kCols = 256;         // key groups per trip
constexpr int kBlockGroups = 16;   // groups per 128-token block
constexpr int kTripBlocks = kCols / kBlockGroups;  // 16 key blocks per trip
constexpr int kSliceBytesA = kRows * 128;          // 128 rows x 64 two-byte channels
constexpr int kSliceBytesB = kCols * 128;
constexpr int kStageBytes = kSliceBytesA + kSliceBytesB;  // 48 KB
constexpr int kStages = 4;
constexpr int kThreads1 = 192;
constexpr int kMmaWarp = 4, kLoadWarp = 5;
constexpr int kSmem1 = kStages * kStageBytes + 256 + 1024;
constexpr int kMaxTrips = kMaxMaskBlocks / kTripBlocks;  // 128 trips = 2048 blocks
constexpr int kStatusSbeWaitGaveUp = 102;

struct SbeParams {
    // Rank-5 tensor maps over (channel, token in group, group, head, batch); box = 64 channels x 1 x
    // 128 (q) or 256 (k) groups.
    alignas(64) CUtensorMap tm_q;
    alignas(64) CUtensorMap tm_k;
    float* partial;   // [pair][groups_pad][trips * 16]  block sums of 2^(s - m_used)
    float* used_max;  // [pair][groups_pad][trips]       m_used, in log2 units
    int pair0;        // first (batch, head) pair of this pass
    int heads, kv_heads;
    int groups, groups_pad, trips;
    int slices;           // K slices per trip: 8 tokens x head_dim / 64
    int slices_per_token; // head_dim / 64
    float scale_log2;
    // Causal form of the reference's golden: the 128 query groups of a thread block (1024 tokens) see the
    // key groups up to the end of their own 1024-token chunk -- the softmax runs over those -- and each
    // query block then ranks the key blocks up to its own.  key_groups: key groups that exist.
    int causal, key_groups;
    int* status;
};

__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int c0, int c1, int c2,
                                            int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}

struct Ring {
    int idx = 0;
    uint32_t phase = 0;
    __device__ __forceinline__ void next() {
        if (++idx == kStages) {
            idx = 0;
            phase ^= 1u;
        }
    }
};

template <int kFmt>  // 1 bf16, 0 fp16
__global__ void __launch_bounds__(kThreads1, 1) sbe_partial_kernel(const __grid_constant__ SbeParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
    const uint32_t bar_base = smem_u32(bars);
    auto bar_full = [&](int s) { return bar_base + 8u * s; };
    auto bar_empty = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto bar_acc_full = [&](int b) { return bar_base + 8u * (2 * kStages + b); };
    auto bar_acc_empty = [&](int b) { return bar_base + 8u * (2 * kStages + 2 + b); };
    constexpr int kNumBars = 2 * kStages + 4;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* abort_site = abort_flag + 1;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g0 = blockIdx.x * kRows;
    const int pair = p.pair0 + blockIdx.y;
    const int head = pair % p.heads, batch = pair / p.heads;
    const int kv_head = head / (p.heads / p.kv_heads);

    // A grid in which one thread block already gave up a wait leaves at once.  The decision is taken
    // once per thread block (all of its threads stay or all leave: the ones that stay set up barriers
    // and tensor memory for the others).
    if (__syncthreads_or(tid == 0 && p.status && *reinterpret_cast<volatile int*>(p.status) != 0)) return;
    // Key groups this thread block's rows take their softmax over, and the trips that cover them.
    const int my_groups = p.causal ? min(p.key_groups, g0 + kRows) : p.groups;
    const int my_trips = (my_groups + kCols - 1) / kCols;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar_full(s), 1);
            mbar_init(bar_empty(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_acc_full(b), 1);
            mbar_init(bar_acc_empty(b), kRows);
        }
        *abort_flag = 0;
        *abort_site = 0;
        fence_mbar_init();
    }
    if (warp == kLoadWarp && lane == 0) {
        tma_prefetch_desc(&p.tm_q);
        tma_prefetch_desc(&p.tm_k);
    }
    if (warp == 0) {
        __syncwarp();
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == kLoadWarp) {
        if (lane == 0) {
            Ring ring;
            int issued = 0;
            bool ok = true;
            for (int trip = 0; trip < my_trips && ok; ++trip) {
                for (int c = 0; c < p.slices && ok; ++c) {
                    ok = mbar_wait(bar_empty(ring.idx), ring.phase ^ 1u, abort_flag, 1);
                    if (!ok) break;
                    const int tok = c / p.slices_per_token, ch = (c - tok * p.slices_per_token) * 64;
                    const uint32_t dst = smem_u32(smem + ring.idx * kStageBytes);
                    mbar_arrive_expect_tx(bar_full(ring.idx), kStageBytes);
                    tma_load_5d(dst, &p.tm_q, bar_full(ring.idx), ch, kGroup - 1 - tok, g0, head, batch);
                    tma_load_5d(dst + kSliceBytesA, &p.tm_k, bar_full(ring.idx), ch, tok, trip * kCols, kv_head, batch);
                    ring.next();
                    ++issued;
                }
            }
            // Before the CTA may exit, every copy this thread started must have landed.
            const int pending = issued < kStages ? issued : kStages;
            for (int i = 0; i < pending; ++i) {
                const int n = issued - 1 - i;
                mbar_wait_drain(bar_full(n % kStages), static_cast<uint32_t>(n / kStages) & 1u);
            }
        }
    } else if (warp == kMmaWarp) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(kFmt, kRows, kCols, false, false);
            const uint32_t a_lo0 = desc_lo(smem_u32(smem), 16);
            const uint32_t b_lo0 = desc_lo(smem_u32(smem + kSliceBytesA), 16);
            constexpr uint32_t kStageStep = kStageBytes >> 4;
            Ring ring;
            bool ok = true;
            for (int trip = 0; trip < my_trips && ok; ++trip) {
                const int buf = trip & 1;
                ok = mbar_wait(bar_acc_empty(buf), (static_cast<uint32_t>(trip >> 1) & 1u) ^ 1u, abort_flag, 10);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d = tmem_base + buf * kCols;
                for (int c = 0; c < p.slices && ok; ++c) {
                    ok = mbar_wait(bar_full(ring.idx), ring.phase, abort_flag, 11);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_lo = a_lo0 + ring.idx * kStageStep, b_lo = b_lo0 + ring.idx * kStageStep;
#pragma unroll
                    for (int k = 0; k < 4; ++k)  // 16 channels = 32 bytes of the 128-byte row per MMA
                        umma_ss_lohi<false>(d, a_lo + 2 * k, b_lo + 2 * k, kDescHiSbo1024, idesc, (c | k) != 0);
                    umma_commit(bar_empty(ring.idx));
                    ring.next();
                }
                if (ok) umma_commit(bar_acc_full(buf));
            }
        }
    } else if (warp < 4) {
        const int g = g0 + warp * 32 + lane;
        const bool row_ok = g < p.groups;
        const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
        float* prow = p.partial + (static_cast<int64_t>(blockIdx.y) * p.groups_pad + g) * (p.trips * kTripBlocks);
        float* mrow = p.used_max + (static_cast<int64_t>(blockIdx.y) * p.groups_pad + g) * p.trips;
        float m_run = -INFINITY;  // running maximum of the raw accumulators
        bool ok = true;
        for (int trip = 0; trip < my_trips && ok; ++trip) {
            const int buf = trip & 1;
            ok = __all_sync(0xffffffffu, mbar_wait(bar_acc_full(buf), static_cast<uint32_t>(trip >> 1) & 1u, abort_flag, 20));
            if (!ok) break;
            tc_fence_after();
            const uint32_t t0 = tmem_base + lane_base + buf * kCols;
            const int valid = min(kCols, my_groups - trip * kCols);  // key groups of this trip that exist (and are seen)
            // Pass 1: the trip's maximum.  The accumulator is read twice rather than held in 256 registers.
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            for (int c0 = 0; c0 < valid; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(t0 + c0, r);
                tmem_wait_ld();
                if (c0 + 32 <= valid) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) mx[i & 3] = fmaxf(mx[i & 3], __uint_as_float(r[i]));
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (c0 + i < valid) mx[i & 3] = fmaxf(mx[i & 3], __uint_as_float(r[i]));
                }
            }
            // scale_log2 > 0, so the maximum of the scaled logits is the scaled maximum.
            m_run = fmaxf(m_run, fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])));
            const float m_used = m_run * p.scale_log2;
            // Pass 2: 2^(s - m_used), summed over each 16 consecutive key groups.
            float sums[kTripBlocks];
#pragma unroll
            for (int j = 0; j < kTripBlocks; ++j) sums[j] = 0.f;
#pragma unroll
            for (int cc = 0; cc < kCols / 32; ++cc) {
                const int c0 = cc * 32;
                if (c0 < valid) {
                    uint32_t r[32];
                    tmem_ld32(t0 + c0, r);
                    tmem_wait_ld();
                    float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
                    if (c0 + 32 <= valid) {
#pragma unroll
                        for (int i = 0; i < 16; i += 2) {
                            a0 += ex2_approx(fmaf(__uint_as_float(r[i]), p.scale_log2, -m_used));
                            a1 += ex2_approx(fmaf(__uint_as_float(r[i + 1]), p.scale_log2, -m_used));
                            b0 += ex2_approx(fmaf(__uint_as_float(r[16 + i]), p.scale_log2, -m_used));
                            b1 += ex2_approx(fmaf(__uint_as_float(r[17 + i]), p.scale_log2, -m_used));
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            if (c0 + i < valid) a0 += ex2_approx(fmaf(__uint_as_float(r[i]), p.scale_log2, -m_used));
                            if (c0 + 16 + i < valid)
                                b0 += ex2_approx(fmaf(__uint_as_float(r[16 + i]), p.scale_log2, -m_used));
                        }
                    }
                    sums[2 * cc] = a0 + a1;
                    sums[2 * cc + 1] = b0 + b1;
                }
            }
            // The accumulator is free for the MMAs of the trip after next.
            tc_fence_before();
            mbar_arrive(bar_acc_empty(buf));
            if (row_ok) {
                float4* dst = reinterpret_cast<float4*>(prow + trip * kTripBlocks);
#pragma unroll
                for (int j = 0; j < kTripBlocks / 4; ++j)
                    dst[j] = make_float4(sums[4 * j], sums[4 * j + 1], sums[4 * j + 2], sums[4 * j + 3]);
                mrow[trip] = m_used;
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
    if (tid == 0 && *abort_flag && p.status) {
        if (atomicCAS(p.status, 0, kStatusSbeWaitGaveUp) == 0) {
            p.status[1] = *abort_site;
            p.status[2] = static_cast<int>(blockIdx.x);
            p.status[3] = static_cast<int>(blockIdx.y);
            p.status[4] = 0;
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Kernel 2: block scores of one query block, the cumulative-mass decision, mask row and count.
// ------------------------------------------------------------------------------------------------
struct SelectParams {
    const float* partial;
    const float* used_max;
    int pair0, heads;
    int groups, groups_pad, trips, blocks;
    int mask_cols;  // row pitch of the mask: blocks rounded up to a multiple of 32
    float threshold;
    int max_keep;   // cap on the kept prefix (row_sparse), or blocks
    int keep_sink, keep_recent;
    int causal, key_groups;
    double row_sparse;  // causal: the cap is int(row_sparse * (blocks up to the row's own)), per row
    int8_t* mask;   // [batch][heads][blocks][mask_cols]
    int32_t* count; // [batch][heads][blocks]
};

constexpr int kThreads2 = 128;

// kPerLane: ceil(blocks / 32) rounded up to a supported size; warp 0 holds the row's scores in
// registers during the search.
template <int kPerLane>
__global__ void __launch_bounds__(kThreads2) sbe_select_kernel(const SelectParams p) {
    __shared__ float factor[kBlockGroups][kMaxTrips];  // 2^(m_used - m_final) / row sum
    __shared__ float score[kMaxMaskBlocks];
    __shared__ float row_sum[kBlockGroups];
    __shared__ uint32_t guard_smem;
    __shared__ int count_smem;
    const int qb = blockIdx.x;
    const int pair = p.pair0 + blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cols = p.trips * kTripBlocks;  // pitch of a partial row
    const int64_t row_base = static_cast<int64_t>(blockIdx.y) * p.groups_pad + static_cast<int64_t>(qb) * kBlockGroups;
    const int nrows = min(kBlockGroups, p.groups - qb * kBlockGroups);
    // Causal: the row's softmax ran over the key groups up to the end of its 1024-token chunk (what kernel 1
    // wrote); the blocks that compete are those up to the row's own.
    const int seen_groups = p.causal ? min(p.key_groups, (qb / (kRows / kBlockGroups) + 1) * kRows) : p.groups;
    const int trips_q = p.causal ? (seen_groups + kCols - 1) / kCols : p.trips;
    const int seen_blocks = p.causal ? (seen_groups + kBlockGroups - 1) / kBlockGroups : p.blocks;
    const int nb = p.causal ? min(qb + 1, seen_blocks) : p.blocks;  // blocks that compete

    for (int i = tid; i < kBlockGroups * p.trips; i += kThreads2) {
        const int r = i / p.trips, t = i - r * p.trips;
        float f = 0.f;
        if (r < nrows && t < trips_q) {
            const float* m = p.used_max + (row_base + r) * p.trips;
            f = ex2_approx(m[t] - m[trips_q - 1]);
        }
        factor[r][t] = f;
    }
    if (tid == 0) count_smem = 0;
    __syncthreads();
    // Row sums: the softmax denominator in units of the final maximum.  Four rows per warp.
    for (int r = warp; r < kBlockGroups; r += kThreads2 / 32) {
        float s = 0.f;
        if (r < nrows) {
            const float* pr = p.partial + (row_base + r) * cols;
            for (int j = lane; j < seen_blocks; j += 32) s += pr[j] * factor[r][j / kTripBlocks];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) row_sum[r] = s;
    }
    __syncthreads();
    for (int i = tid; i < kBlockGroups * p.trips; i += kThreads2) {
        const int r = i / p.trips, t = i - r * p.trips;
        if (r < nrows) factor[r][t] = factor[r][t] / row_sum[r];
    }
    __syncthreads();
    for (int j = tid; j < nb; j += kThreads2) {
        const int t = j / kTripBlocks;
        float s = 0.f;
        for (int r = 0; r < nrows; ++r) s += p.partial[(row_base + r) * cols + j] * factor[r][t];
        // The last block does not compete: kept anyway (keep_recent), or -- causal -- the row's own block,
        // whose mass the golden clears before ranking.
        if ((p.keep_recent || p.causal) && j == nb - 1) s = 0.f;
        score[j] = s;
    }
    int max_keep = p.max_keep;
    if (p.causal) {
        max_keep = nb;
        if (p.row_sparse > 0.0 && p.row_sparse * nb < nb) max_keep = max(1, static_cast<int>(p.row_sparse * nb));
    }
    __syncthreads();
    // The guard is the score of the block at which the running sum of the descending scores first reaches
    // `threshold` of the total: the largest score v for which the blocks scoring at least v hold that
    // much -- or, if that takes more than max_keep blocks, the max_keep-th largest score.  Both
    // conditions are monotone in v, so the guard is found bit by bit on the scores' bit patterns
    // (non-negative floats order like unsigned integers) without sorting.
    if (warp == 0) {
        float x[kPerLane];
        float total = 0.f;
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) {
            const int j = lane + 32 * i;
            x[i] = j < nb ? score[j] : -1.f;  // padding never reaches a candidate
            total += fmaxf(x[i], 0.f);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
        const float limit = p.threshold * total;
        uint32_t thr = 0;
        // Causal rows 0 and 1 keep every block up to their own (guard 0).
        if (total > 0.f && !(p.causal && qb <= 1)) {
            for (int bit = 30; bit >= 0; --bit) {
                const uint32_t cand = thr | (1u << bit);
                float mass = 0.f;
                int cnt = 0;
#pragma unroll
                for (int i = 0; i < kPerLane; ++i) {
                    const bool ge = x[i] >= 0.f && __float_as_uint(x[i]) >= cand;
                    mass += ge ? x[i] : 0.f;
                    cnt += ge;
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) mass += __shfl_xor_sync(0xffffffffu, mass, o);
                cnt = __reduce_add_sync(0xffffffffu, cnt);
                if (mass >= limit || cnt >= max_keep) thr = cand;
            }
        }
        if (lane == 0) guard_smem = thr;
    }
    __syncthreads();
    const uint32_t guard = guard_smem;
    int8_t* mrow = p.mask + (static_cast<int64_t>(pair) * p.blocks + qb) * p.mask_cols;
    int kept = 0;
    for (int j = tid; j < p.mask_cols; j += kThreads2) {
        bool keep = false;
        if (j < nb)
            keep = __float_as_uint(score[j]) >= guard || (p.keep_sink && j == 0) ||
                   (!p.causal && p.keep_recent && j == p.blocks - 1);
        mrow[j] = keep ? 1 : 0;
        kept += keep;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) kept += __shfl_xor_sync(0xffffffffu, kept, o);
    if (lane == 0 && kept) atomicAdd(&count_smem, kept);
    __syncthreads();
    if (tid == 0) p.count[static_cast<int64_t>(pair) * p.blocks + qb] = count_smem;
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn5() {
    static EncodeFn fn = [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess) sym = nullptr;
        return reinterpret_cast<EncodeFn>(sym);
    }();
    return fn;
}

// Rank-5 map over (channel, token in group, group, head, batch) of a [batch, head, token, channel] tensor.
int encode_group_map(CUtensorMap* map, const void* base, int dtype, int channels, int64_t groups, int heads, int batch,
                     const int64_t stride[3], int box_groups) {
    EncodeFn fn = encode_fn5();
    if (!fn) return MINDIESD_E_DRIVER;
    if (reinterpret_cast<uintptr_t>(base) % 16) return MINDIESD_E_STRIDE;
    for (int i = 0; i < 3; ++i)
        if (stride[i] < 0 || (stride[i] * 2) % 16) return MINDIESD_E_STRIDE;
    if (stride[2] <= 0) return MINDIESD_E_STRIDE;
    const int64_t tok = stride[2];
    auto bytes = [&](int64_t s, int64_t fallback) { return static_cast<cuuint64_t>((s > 0 ? s : fallback) * 2); };
    const cuuint64_t dims[5] = {static_cast<cuuint64_t>(channels), kGroup, static_cast<cuuint64_t>(groups),
                                static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(batch)};
    const cuuint64_t strides[4] = {bytes(tok, 0), bytes(tok * kGroup, 0), bytes(stride[1], tok * kGroup * groups),
                                   bytes(stride[0], tok * kGroup * groups * heads)};
    const cuuint32_t box[5] = {64, 1, static_cast<cuuint32_t>(box_groups), 1, 1};
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    const CUresult r = fn(map, dtype == MINDIESD_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5,
                          const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? MINDIESD_OK : MINDIESD_E_DRIVER;
}

struct Sizes {
    int groups, groups_pad, trips, blocks;
    size_t per_pair;  // scratch bytes of one (batch, head) pair
};

Sizes sizes_of(int seq) {
    Sizes s;
    s.groups = seq / kGroup;
    s.groups_pad = (s.groups + kRows - 1) / kRows * kRows;
    s.trips = (s.groups + kCols - 1) / kCols;
    s.blocks = (seq + 127) / 128;
    s.per_pair = static_cast<size_t>(s.groups_pad) * (s.trips * kTripBlocks + s.trips) * sizeof(float);
    return s;
}

constexpr int kPairsPerPass = 4;  // the partial sums of four heads at 75 600 tokens (95 MB) stay in L2

}  // namespace

}  // namespace sdb

using namespace sdb;

extern "C" size_t mindiesd_sparse_block_estimate_scratch_bytes(int32_t batch, int32_t heads, int32_t seq) {
    if (batch <= 0 || heads <= 0 || seq <= 0) return 0;
    const Sizes s = sizes_of(seq);
    const int64_t pairs = static_cast<int64_t>(batch) * heads;
    return s.per_pair * static_cast<size_t>(pairs < kPairsPerPass ? pairs : kPairsPerPass);
}

extern "C" int mindiesd_sparse_block_estimate(const mindiesd_estimate_args* a, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!a || !a->q || !a->k || !a->mask || !a->count || !a->scratch) return MINDIESD_E_NULL;
    if (a->dtype != MINDIESD_BF16 && a->dtype != MINDIESD_FP16) return MINDIESD_E_DTYPE;
    if (a->batch <= 0 || a->heads <= 0 || a->kv_heads <= 0 || a->heads % a->kv_heads || a->seq <= 0) return MINDIESD_E_SHAPE;
    if (a->head_dim != 64 && a->head_dim != 128) return MINDIESD_E_SHAPE;
    if (a->stride != kGroup || a->sparse_size != 128) return MINDIESD_E_SHAPE;
    if (a->seq % kGroup) return MINDIESD_E_SHAPE;  // the caller pads the token axis with zeros
    if (a->causal && (a->causal_key_tokens < 0 || a->causal_key_tokens > a->seq)) return MINDIESD_E_VALUE;
    if (!(a->scale > 0.0f) || !(a->threshold >= 0.0f) || !(a->row_sparse >= 0.0)) return MINDIESD_E_VALUE;
    const Sizes s = sizes_of(a->seq);
    if (s.blocks > kMaxMaskBlocks) return MINDIESD_E_CAPACITY;
    if (a->mask_cols < s.blocks) return MINDIESD_E_SHAPE;
    if (a->scratch_bytes < s.per_pair || reinterpret_cast<uintptr_t>(a->scratch) % 16) return MINDIESD_E_CAPACITY;

    SbeParams p;
    int rc;
    if ((rc = encode_group_map(&p.tm_q, a->q, a->dtype, a->head_dim, s.groups, a->heads, a->batch, a->q_stride, kRows))) return rc;
    if ((rc = encode_group_map(&p.tm_k, a->k, a->dtype, a->head_dim, s.groups, a->kv_heads, a->batch, a->k_stride, kCols))) return rc;
    const int64_t pairs = static_cast<int64_t>(a->batch) * a->heads;
    int64_t per_pass = static_cast<int64_t>(a->scratch_bytes / s.per_pair);
    if (per_pass > kPairsPerPass) per_pass = kPairsPerPass;
    p.partial = static_cast<float*>(a->scratch);
    p.used_max = p.partial + static_cast<size_t>(per_pass) * s.groups_pad * s.trips * kTripBlocks;
    p.heads = a->heads;
    p.kv_heads = a->kv_heads;
    p.groups = s.groups;
    p.groups_pad = s.groups_pad;
    p.trips = s.trips;
    p.slices_per_token = a->head_dim / 64;
    p.slices = kGroup * p.slices_per_token;
    p.scale_log2 = a->scale * 1.4426950408889634f;
    p.causal = a->causal != 0;
    p.key_groups = (a->causal && a->causal_key_tokens > 0 ? a->causal_key_tokens : a->seq) / kGroup;
    p.status = device_status_word();

    SelectParams sp;
    sp.partial = p.partial;
    sp.used_max = p.used_max;
    sp.heads = a->heads;
    sp.groups = s.groups;
    sp.groups_pad = s.groups_pad;
    sp.trips = s.trips;
    sp.blocks = s.blocks;
    sp.mask_cols = a->mask_cols;
    sp.threshold = a->threshold;
    sp.max_keep = s.blocks;
    // The reference caps the kept prefix at int(row_sparse * blocks) when the prefix is longer than
    // row_sparse * blocks (a comparison in double precision).
    if (a->row_sparse > 0.0 && a->row_sparse * s.blocks < s.blocks) {
        sp.max_keep = static_cast<int>(a->row_sparse * s.blocks);
        if (sp.max_keep < 1) sp.max_keep = 1;
    }
    sp.keep_sink = a->keep_sink ? 1 : 0;
    sp.keep_recent = a->keep_recent ? 1 : 0;
    sp.causal = p.causal;
    sp.key_groups = p.key_groups;
    sp.row_sparse = a->row_sparse;
    sp.mask = a->mask;
    sp.count = a->count;

    auto kernel = a->dtype == MINDIESD_BF16 ? sbe_partial_kernel<1> : sbe_partial_kernel<0>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem1);
    if (e != cudaSuccess) return static_cast<int>(e);
    for (int64_t pair0 = 0; pair0 < pairs; pair0 += per_pass) {
        const int n = static_cast<int>(pairs - pair0 < per_pass ? pairs - pair0 : per_pass);
        p.pair0 = sp.pair0 = static_cast<int>(pair0);
        kernel<<<dim3(s.groups_pad / kRows, n), kThreads1, kSmem1, stream>>>(p);
        if ((e = cudaGetLastError()) != cudaSuccess) return static_cast<int>(e);
        const dim3 grid2(s.blocks, n);
        const int per_lane = (s.blocks + 31) / 32;
        if (per_lane <= 8) sbe_select_kernel<8><<<grid2, kThreads2, 0, stream>>>(sp);
        else if (per_lane <= 20) sbe_select_kernel<20><<<grid2, kThreads2, 0, stream>>>(sp);
        else if (per_lane <= 32) sbe_select_kernel<32><<<grid2, kThreads2, 0, stream>>>(sp);
        else sbe_select_kernel<64><<<grid2, kThreads2, 0, stream>>>(sp);
        if ((e = cudaGetLastError()) != cudaSuccess) return static_cast<int>(e);
    }
    return MINDIESD_OK;
}

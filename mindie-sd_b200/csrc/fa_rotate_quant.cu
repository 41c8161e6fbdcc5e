// Rotation by a learned 128x128 matrix fused with the e4m3 block quantisation of an attention operand.
//
// y = x R for every token (x: [B, N, S, 128] bf16/fp16, R: 128x128 in the same type), then one scale per
// (row_block tokens x 128 channels) block, scale = absmax(y) / 448, and y / scale cast to e4m3.  Unfused
// this is a GEMM that writes y (2 bytes per element) and a quantiser that reads it back; fused, y never
// leaves the SM: 2 bytes in, 1 byte out per element.
//
// Two forms.  128-token quantisation blocks (the layer's choice) run as a persistent pipeline, one CTA per
// SM: R is fetched once, a loader thread keeps four 128-token tiles in flight, an MMA thread issues eight
// tcgen05 MMAs (M128 N128 K16) per tile into one of four 128-column accumulators, and two groups of four
// warps take alternate tiles: read the accumulator once (one token per thread, the 128 products stay in
// registers), reduce the block's absolute maximum, scale, convert, store.  Loads, MMAs and the two
// groups' passes overlap across tiles.  256- and 512-token blocks run one CTA per block: all of the
// block's tiles are multiplied first and the accumulators are read twice (maximum, then conversion).
// R is the B operand in its natural [k][n] layout (n contiguous), the layout V has in the attention kernel.
#include "capi_common.h"
#include "ptx_sm100.cuh"

namespace sdb {

namespace {

constexpr int kTile = 128;
constexpr int kAtomBytes = kTile * 128;     // 128 rows of one 64-channel (128-byte) swizzle atom
constexpr int kTileBytes = 2 * kAtomBytes;  // 32 KB: a 128 x 128 two-byte tile
constexpr int kThreads = 160;
constexpr int kIssueWarp = 4;
constexpr int kStatusRotqWaitGaveUp = 103;

struct RotqParams {
    alignas(64) CUtensorMap tm_x;  // (channel, token, head, batch), box 64 x 128
    alignas(64) CUtensorMap tm_r;  // (n, k, 1, 1), box 64 x 128
    uint8_t* out;                  // e4m3 [B, N, S, 128] contiguous
    float* scales;                 // [B, N, blocks]
    int heads, seq, blocks;
    float post_scale;              // the stored scale is absmax / 448 * post_scale (1, or 1/sqrt(128) for the +-1 matrix)
    int* status;
};

// The 128-point Sylvester Hadamard matrix with entries +-1 as bf16 and as fp16 bit patterns: exact in
// both types, so the rotation it applies is sqrt(128) times an exactly orthogonal one and the factor
// goes into the stored scale.
struct HadamardTables {
    uint16_t bf16[128 * 128];
    uint16_t fp16[128 * 128];
    constexpr HadamardTables() : bf16(), fp16() {
        for (int i = 0; i < 128; ++i)
            for (int j = 0; j < 128; ++j) {
                int v = i & j, parity = 0;
                while (v) {
                    parity ^= v & 1;
                    v >>= 1;
                }
                bf16[i * 128 + j] = parity ? 0xBF80 : 0x3F80;
                fp16[i * 128 + j] = parity ? 0xBC00 : 0x3C00;
            }
    }
};
__device__ const HadamardTables g_hadamard = HadamardTables();

__device__ __forceinline__ uint32_t pack_quad_e4m3(float a, float b, float c, float d) {
    uint16_t lo, hi;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
    return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

// kFmt: 1 bf16, 0 fp16.  kTiles: 128-token tiles per quantisation block (1, 2 or 4).
template <int kFmt, int kTiles>
__global__ void __launch_bounds__(kThreads) rotq_kernel(const __grid_constant__ RotqParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sm_r = smem;
    uint8_t* sm_x = smem + kTileBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm_x + kTiles * kTileBytes);
    const uint32_t bar_base = smem_u32(bars);
    auto bar_r = [&]() { return bar_base; };
    auto bar_x = [&](int i) { return bar_base + 8u * (1 + i); };
    auto bar_d = [&](int i) { return bar_base + 8u * (1 + kTiles + i); };
    constexpr int kNumBars = 1 + 2 * kTiles;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* abort_site = abort_flag + 1;
    float* warp_max = reinterpret_cast<float*>(tmem_slot + 4);
    constexpr uint32_t kTmemCols = 128 * kTiles;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int blk = blockIdx.x, head = blockIdx.y, batch = blockIdx.z;
    const int row0 = blk * kTiles * kTile;

    // A grid in which one thread block already gave up a wait leaves at once.  The decision is taken
    // once per thread block (all of its threads stay or all leave: the ones that stay set up barriers
    // and tensor memory for the others).
    if (__syncthreads_or(tid == 0 && p.status && *reinterpret_cast<volatile int*>(p.status) != 0)) return;

    if (tid == 0) {
        for (int i = 0; i < kNumBars; ++i) mbar_init(bar_base + 8u * i, 1);
        *abort_flag = 0;
        *abort_site = 0;
        fence_mbar_init();
    }
    if (warp == kIssueWarp && lane == 0) {
        tma_prefetch_desc(&p.tm_x);
        tma_prefetch_desc(&p.tm_r);
    }
    if (warp == 0) {
        __syncwarp();
        tmem_alloc(smem_u32(tmem_slot), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == kIssueWarp) {
        if (lane == 0) {
            mbar_arrive_expect_tx(bar_r(), kTileBytes);
            for (int a = 0; a < 2; ++a) tma_load_4d(smem_u32(sm_r + a * kAtomBytes), &p.tm_r, bar_r(), a * 64, 0, 0, 0);
            for (int i = 0; i < kTiles; ++i) {
                mbar_arrive_expect_tx(bar_x(i), kTileBytes);
                for (int a = 0; a < 2; ++a)
                    tma_load_4d(smem_u32(sm_x + i * kTileBytes + a * kAtomBytes), &p.tm_x, bar_x(i), a * 64,
                                row0 + i * kTile, head, batch);
            }
            const uint32_t idesc = umma_idesc(kFmt, kTile, kTile, false, true);
            const uint32_t r_lo = desc_lo(smem_u32(sm_r), kAtomBytes);  // MN-major: 16 KB between the 64-column atoms
            bool ok = mbar_wait(bar_r(), 0, abort_flag, 1);
            if (!ok) mbar_wait_drain(bar_r(), 0);
            for (int i = 0; i < kTiles; ++i) {
                // Every started copy is waited for, also after a wait has given up.
                const bool landed = ok ? mbar_wait(bar_x(i), 0, abort_flag, 2) : mbar_wait_drain(bar_x(i), 0);
                ok = ok && landed;
                if (!ok) continue;
                tc_fence_after();
                const uint32_t x_lo = desc_lo(smem_u32(sm_x + i * kTileBytes), 16);
#pragma unroll
                for (int kc = 0; kc < 8; ++kc) {  // 16 channels of x = 16 rows of R per MMA
                    const uint32_t a_off = (kc >> 2) * (kAtomBytes >> 4) + (kc & 3) * 2;
                    const uint32_t b_off = kc * (16 * 128 >> 4);
                    umma_ss_lohi<false>(tmem_base + i * kTile, x_lo + a_off, r_lo + b_off, kDescHiSbo1024, idesc, kc > 0);
                }
                umma_commit(bar_d(i));
            }
        }
    } else {
        const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
        // Pass 1: absolute maximum of the block.
        float mx = 0.0f;
        bool ok = true;
        for (int i = 0; i < kTiles && ok; ++i) {
            ok = __all_sync(0xffffffffu, mbar_wait(bar_d(i), 0, abort_flag, 10));
            if (!ok) break;
            tc_fence_after();
            float m4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                tmem_ld32(tmem_base + lane_base + i * kTile + c * 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 32; ++j) m4[j & 3] = fmaxf(m4[j & 3], fabsf(__uint_as_float(r[j])));
            }
            mx = fmaxf(mx, fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (lane == 0) warp_max[warp] = mx;
        asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps only
        const float amax = fmaxf(fmaxf(warp_max[0], warp_max[1]), fmaxf(warp_max[2], warp_max[3]));
        const float scale = amax > 0.0f ? amax / 448.0f : 1.0f;
        const float inv = 1.0f / scale;
        if (tid == 0 && ok) p.scales[(static_cast<int64_t>(batch) * p.heads + head) * p.blocks + blk] = scale * p.post_scale;
        // Pass 2: scale, convert, store (128 bytes per token).
        for (int i = 0; i < kTiles && ok; ++i) {
            const int row = row0 + i * kTile + warp * 32 + lane;
            uint4* dst = reinterpret_cast<uint4*>(p.out + ((static_cast<int64_t>(batch) * p.heads + head) * p.seq + row) * 128);
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                tmem_ld32(tmem_base + lane_base + i * kTile + c * 32, r);
                tmem_wait_ld();
                uint32_t w[8];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    w[j] = pack_quad_e4m3(__uint_as_float(r[4 * j]) * inv, __uint_as_float(r[4 * j + 1]) * inv,
                                          __uint_as_float(r[4 * j + 2]) * inv, __uint_as_float(r[4 * j + 3]) * inv);
                if (row < p.seq) {
                    dst[2 * c] = make_uint4(w[0], w[1], w[2], w[3]);
                    dst[2 * c + 1] = make_uint4(w[4], w[5], w[6], w[7]);
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
    if (tid == 0 && *abort_flag && p.status) {
        if (atomicCAS(p.status, 0, kStatusRotqWaitGaveUp) == 0) {
            p.status[1] = *abort_site;
            p.status[2] = static_cast<int>(blockIdx.x);
            p.status[3] = static_cast<int>(blockIdx.y);
            p.status[4] = static_cast<int>(blockIdx.z);
        }
    }
}

// OR of a predicate over the 128 threads that meet at named barrier `id` (one epilogue group).
__device__ __forceinline__ bool group_or(int id, bool pred) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "bar.red.or.pred p, %2, 128, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r)
        : "r"(static_cast<uint32_t>(pred)), "r"(id)
        : "memory");
    return r != 0;
}

// ---- persistent form, 128-token blocks ---------------------------------------------------------------
constexpr int kPThreads = 320;  // warps 0-3 and 4-7: the two epilogue groups; warp 8: loader; warp 9: MMA
constexpr int kPStages = 4;     // tiles of x in flight
constexpr int kPAcc = 4;        // accumulators (128 columns each: all of tensor memory)

template <int kFmt>
__global__ void __launch_bounds__(kPThreads, 1) rotq_persistent_kernel(const __grid_constant__ RotqParams p, int items) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sm_r = smem;
    uint8_t* sm_x = smem + kTileBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm_x + kPStages * kTileBytes);
    const uint32_t bar_base = smem_u32(bars);
    auto bar_r = [&]() { return bar_base; };
    auto x_full = [&](int i) { return bar_base + 8u * (1 + i); };
    auto x_empty = [&](int i) { return bar_base + 8u * (1 + kPStages + i); };
    auto acc_full = [&](int i) { return bar_base + 8u * (1 + 2 * kPStages + i); };
    auto acc_empty = [&](int i) { return bar_base + 8u * (1 + 2 * kPStages + kPAcc + i); };
    auto bar_done = [&]() { return bar_base + 8u * (1 + 2 * kPStages + 2 * kPAcc); };
    constexpr int kNumBars = 2 + 2 * kPStages + 2 * kPAcc;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* abort_site = abort_flag + 1;
    float* warp_max = reinterpret_cast<float*>(tmem_slot + 4);  // [group][parity][warp]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // tiles of this CTA: blockIdx.x, blockIdx.x + gridDim.x, ...; tile w = block + blocks * (head + heads * batch)
    const int my_items = items > static_cast<int>(blockIdx.x) ? (items - 1 - static_cast<int>(blockIdx.x)) / static_cast<int>(gridDim.x) + 1 : 0;
    auto where = [&](int i, int& blk, int& head, int& batch) {
        const int w = static_cast<int>(blockIdx.x) + i * static_cast<int>(gridDim.x);
        blk = w % p.blocks;
        const int hb = w / p.blocks;
        head = hb % p.heads;
        batch = hb / p.heads;
    };

    if (__syncthreads_or(tid == 0 && p.status && *reinterpret_cast<volatile int*>(p.status) != 0)) return;

    if (tid == 0) {
        mbar_init(bar_r(), 1);
        for (int i = 0; i < kPStages; ++i) {
            mbar_init(x_full(i), 1);
            mbar_init(x_empty(i), 1);
        }
        for (int i = 0; i < kPAcc; ++i) {
            mbar_init(acc_full(i), 1);
            mbar_init(acc_empty(i), 128);
        }
        mbar_init(bar_done(), 1);
        *abort_flag = 0;
        *abort_site = 0;
        fence_mbar_init();
    }
    if (warp == 8 && lane == 0) {
        tma_prefetch_desc(&p.tm_x);
        tma_prefetch_desc(&p.tm_r);
    }
    if (warp == 0) {
        __syncwarp();
        tmem_alloc(smem_u32(tmem_slot), 128 * kPAcc);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 8) {
        // ---- loader ----
        if (lane == 0) {
            mbar_arrive_expect_tx(bar_r(), kTileBytes);
            for (int a = 0; a < 2; ++a) tma_load_4d(smem_u32(sm_r + a * kAtomBytes), &p.tm_r, bar_r(), a * 64, 0, 0, 0);
            int issued = 0;
            for (int i = 0; i < my_items; ++i) {
                const int s = i % kPStages;
                if (!mbar_wait(x_empty(s), ((i / kPStages) & 1) ^ 1u, abort_flag, 1)) break;
                int blk, head, batch;
                where(i, blk, head, batch);
                mbar_arrive_expect_tx(x_full(s), kTileBytes);
                for (int a = 0; a < 2; ++a)
                    tma_load_4d(smem_u32(sm_x + s * kTileBytes + a * kAtomBytes), &p.tm_x, x_full(s), a * 64, blk * kTile,
                                head, batch);
                ++issued;
            }
            // Every started copy is waited for before the CTA may exit.
            mbar_wait_drain(bar_r(), 0);
            const int pending = issued < kPStages ? issued : kPStages;
            for (int k = 0; k < pending; ++k) {
                const int n = issued - 1 - k;
                mbar_wait_drain(x_full(n % kPStages), static_cast<uint32_t>(n / kPStages) & 1u);
            }
        }
    } else if (warp == 9) {
        // ---- MMA issue ----
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(kFmt, kTile, kTile, false, true);
            const uint32_t r_lo = desc_lo(smem_u32(sm_r), kAtomBytes);  // MN-major: 16 KB between the 64-column atoms
            bool ok = mbar_wait(bar_r(), 0, abort_flag, 2);
            for (int i = 0; ok && i < my_items; ++i) {
                const int s = i % kPStages, a = i % kPAcc;
                ok = mbar_wait(x_full(s), (i / kPStages) & 1u, abort_flag, 3);
                if (!ok) break;
                ok = mbar_wait(acc_empty(a), ((i / kPAcc) & 1) ^ 1u, abort_flag, 4);
                if (!ok) break;
                tc_fence_after();
                const uint32_t x_lo = desc_lo(smem_u32(sm_x + s * kTileBytes), 16);
#pragma unroll
                for (int kc = 0; kc < 8; ++kc) {  // 16 channels of x = 16 rows of R per MMA
                    const uint32_t a_off = (kc >> 2) * (kAtomBytes >> 4) + (kc & 3) * 2;
                    const uint32_t b_off = kc * (16 * 128 >> 4);
                    umma_ss_lohi<false>(tmem_base + a * kTile, x_lo + a_off, r_lo + b_off, kDescHiSbo1024, idesc, kc > 0);
                }
                umma_commit(acc_full(a));
                umma_commit(x_empty(s));
            }
            // Tensor memory is freed at the end: every product issued must be over by then.
            umma_commit(bar_done());
            mbar_wait_drain(bar_done(), 0);
        }
    } else {
        // ---- epilogue groups: tiles g, g + 2, ... ----
        const int g = warp >> 2, wg = warp & 3;
        const uint32_t lane_base = static_cast<uint32_t>(wg * 32) << 16;
        for (int i = g; i < my_items; i += 2) {
            const int a = i % kPAcc;
            // The four warps of a group stay together: they meet at a barrier below, so a wait that gave up in
            // one of them takes all of them out of the loop.
            const bool gave_up = !__all_sync(0xffffffffu, mbar_wait(acc_full(a), (i / kPAcc) & 1u, abort_flag, 10 + g));
            if (group_or(1 + g, gave_up)) break;
            tc_fence_after();
            uint32_t r[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld32(tmem_base + lane_base + a * kTile + c * 32, r[c]);
            tmem_wait_ld();
            // the accumulator is in registers: the MMA thread may reuse it
            tc_fence_before();
            mbar_arrive(acc_empty(a));
            float m4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int j = 0; j < 32; ++j) m4[j & 3] = fmaxf(m4[j & 3], fabsf(__uint_as_float(r[c][j])));
            float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            float* wm = warp_max + (g * 2 + ((i >> 1) & 1)) * 4;  // alternate buffers: the previous tile's may still be read
            if (lane == 0) wm[wg] = mx;
            if (g == 0) asm volatile("bar.sync 3, 128;" ::: "memory");
            else asm volatile("bar.sync 4, 128;" ::: "memory");
            const float amax = fmaxf(fmaxf(wm[0], wm[1]), fmaxf(wm[2], wm[3]));
            const float scale = amax > 0.0f ? amax / 448.0f : 1.0f;
            const float inv = 1.0f / scale;
            int blk, head, batch;
            where(i, blk, head, batch);
            if (wg == 0 && lane == 0) p.scales[(static_cast<int64_t>(batch) * p.heads + head) * p.blocks + blk] = scale * p.post_scale;
            const int row = blk * kTile + wg * 32 + lane;
            if (row < p.seq) {
                uint4* dst = reinterpret_cast<uint4*>(p.out + ((static_cast<int64_t>(batch) * p.heads + head) * p.seq + row) * 128);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t w[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        w[j] = pack_quad_e4m3(__uint_as_float(r[c][4 * j]) * inv, __uint_as_float(r[c][4 * j + 1]) * inv,
                                              __uint_as_float(r[c][4 * j + 2]) * inv, __uint_as_float(r[c][4 * j + 3]) * inv);
                    dst[2 * c] = make_uint4(w[0], w[1], w[2], w[3]);
                    dst[2 * c + 1] = make_uint4(w[4], w[5], w[6], w[7]);
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 128 * kPAcc);
    }
    if (tid == 0 && *abort_flag && p.status) {
        if (atomicCAS(p.status, 0, kStatusRotqWaitGaveUp) == 0) {
            p.status[1] = *abort_site;
            p.status[2] = static_cast<int>(blockIdx.x);
            p.status[3] = 0;
            p.status[4] = 0;
        }
    }
}

template <int kFmt>
cudaError_t launch_rotq_persistent(const RotqParams& p, int batch, cudaStream_t stream) {
    const int smem = (1 + kPStages) * kTileBytes + 512 + 1024;
    cudaError_t e = cudaFuncSetAttribute(rotq_persistent_kernel<kFmt>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    const int64_t items = static_cast<int64_t>(p.blocks) * p.heads * batch;
    if (items > 0x7fffffff) return cudaErrorInvalidValue;
    static const int sms = [] {
        int dev = 0, n = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        return n > 0 ? n : 148;
    }();
    const int grid = items < sms ? static_cast<int>(items) : sms;
    rotq_persistent_kernel<kFmt><<<grid, kPThreads, smem, stream>>>(p, static_cast<int>(items));
    return cudaGetLastError();
}

template <int kFmt, int kTiles>
cudaError_t launch_rotq(const RotqParams& p, dim3 grid, cudaStream_t stream) {
    const int smem = (1 + kTiles) * kTileBytes + 256 + 1024;
    cudaError_t e = cudaFuncSetAttribute(rotq_kernel<kFmt, kTiles>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    rotq_kernel<kFmt, kTiles><<<grid, kThreads, smem, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace

int rotate_quant_launch(const void* x, const int64_t x_stride[3], const void* rot, int dtype, int batch, int heads, int seq,
                        int row_block, void* out, float* scales, float post_scale, cudaStream_t stream) {
    if (reinterpret_cast<uintptr_t>(out) % 16) return MINDIESD_E_STRIDE;
    RotqParams p;
    int rc;
    if ((rc = encode_tile_map(&p.tm_x, x, dtype, 128, seq, heads, batch, x_stride, 128))) return rc;
    const int64_t r_stride[3] = {0, 0, 128};
    if ((rc = encode_tile_map(&p.tm_r, rot, dtype, 128, 128, 1, 1, r_stride, 128))) return rc;
    p.out = static_cast<uint8_t*>(out);
    p.scales = scales;
    p.heads = heads;
    p.seq = seq;
    p.blocks = (seq + row_block - 1) / row_block;
    p.post_scale = post_scale;
    p.status = device_status_word();
    const dim3 grid(p.blocks, heads, batch);
    const bool bf16 = dtype == MINDIESD_BF16;
    cudaError_t e;
    if (row_block == 128) e = bf16 ? launch_rotq_persistent<1>(p, batch, stream) : launch_rotq_persistent<0>(p, batch, stream);
    else if (row_block == 256) e = bf16 ? launch_rotq<1, 2>(p, grid, stream) : launch_rotq<0, 2>(p, grid, stream);
    else e = bf16 ? launch_rotq<1, 4>(p, grid, stream) : launch_rotq<0, 4>(p, grid, stream);
    return e == cudaSuccess ? MINDIESD_OK : static_cast<int>(e);
}

int hadamard_quant_launch(const void* x, const int64_t x_stride[3], int dtype, int batch, int heads, int seq, int row_block,
                          void* out, float* scales, cudaStream_t stream) {
    void* sym = nullptr;
    if (cudaGetSymbolAddress(&sym, g_hadamard) != cudaSuccess || !sym) return MINDIESD_E_DRIVER;
    const HadamardTables* tables = static_cast<const HadamardTables*>(sym);
    const void* rot = dtype == MINDIESD_BF16 ? static_cast<const void*>(tables->bf16) : static_cast<const void*>(tables->fp16);
    return rotate_quant_launch(x, x_stride, rot, dtype, batch, heads, seq, row_block, out, scales, 0.08838834764831845f, stream);
}

}  // namespace sdb

using namespace sdb;

extern "C" int mindiesd_fa_rotate_quant(const mindiesd_rotate_quant_args* a, void* stream_) {
    if (!a || !a->x || !a->rot || !a->out || !a->scales) return MINDIESD_E_NULL;
    if (a->head_dim != 128) return MINDIESD_E_SHAPE;
    if (a->batch <= 0 || a->heads <= 0 || a->seq <= 0) return MINDIESD_E_SHAPE;
    if (a->batch > 65535 || a->heads > 65535) return MINDIESD_E_SHAPE;
    if (a->dtype != MINDIESD_BF16 && a->dtype != MINDIESD_FP16) return MINDIESD_E_DTYPE;
    if (a->row_block != 128 && a->row_block != 256 && a->row_block != 512) return MINDIESD_E_SHAPE;
    return rotate_quant_launch(a->x, a->x_stride, a->rot, a->dtype, a->batch, a->heads, a->seq, a->row_block, a->out,
                               a->scales, 1.0f, static_cast<cudaStream_t>(stream_));
}

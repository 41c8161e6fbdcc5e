// RainFusion host-logic replacements, all HBM-bound byte/index work:
//   * token permutation into 8x8 spatial windows and back (gather of 16-byte vectors),
//   * pooled block means of the permuted q and k, read straight from the un-permuted tensors,
//   * block scores, k-th-largest threshold per row and the int8 mask / compacted block lists.
#include "capi_common.h"
#include "rf_grid.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace sdb {

namespace {

// ------------------------------------------------------------------------------------------------
// Permutation: one 16-byte vector per thread, consecutive threads along the channel dimension.
// ------------------------------------------------------------------------------------------------
struct RearrangeParams {
    const uint4* src;
    uint4* dst;
    int64_t src_stride[3], dst_stride[3];  // in 16-byte vectors: batch, head, token
    int heads, seq, vec_per_row;
    Grid g;
    int inverse;
};

constexpr int kRearrangeRows = 128;  // token rows one CTA moves

__global__ void __launch_bounds__(256) rf_rearrange_kernel(const RearrangeParams p) {
    // The source index of a position costs several integer divisions: it is computed once per row
    // (not once per 16-byte lane) and shared through shared memory.
    __shared__ int src_tok[kRearrangeRows];
    const int head = blockIdx.y % p.heads;
    const int batch = blockIdx.y / p.heads;
    const int pos0 = blockIdx.x * kRearrangeRows;  // first position (permuted order) of this CTA
    const int nrows = min(kRearrangeRows, p.seq - pos0);
    if (threadIdx.x < nrows) src_tok[threadIdx.x] = source_of(p.g, pos0 + threadIdx.x);
    __syncthreads();
    const uint4* src = p.src + batch * p.src_stride[0] + head * p.src_stride[1];
    uint4* dst = p.dst + batch * p.dst_stride[0] + head * p.dst_stride[1];
    const int total = nrows * p.vec_per_row;
    // Four vectors per thread and trip: the loads are issued before the stores.
    for (int i0 = threadIdx.x; i0 < total; i0 += 4 * 256) {
        uint4 val[4];
        int64_t to[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * 256;
            if (i < total) {
                const int r = i / p.vec_per_row, v = i - r * p.vec_per_row;
                const int a = pos0 + r, b = src_tok[r];
                val[u] = src[static_cast<int64_t>(p.inverse ? a : b) * p.src_stride[2] + v];
                to[u] = static_cast<int64_t>(p.inverse ? b : a) * p.dst_stride[2] + v;
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (i0 + u * 256 < total) dst[to[u]] = val[u];
    }
}

// ------------------------------------------------------------------------------------------------
// Pooled means.  Grid: (block, head, batch * ntensors) -- with two tensors the low bit of the last
// index selects q or k.
// A block is up to 128 consecutive positions of the permuted image, or of the text; image and
// text are pooled separately, so the last image block and the last text block may be short.
// Sums are exact in fp64 (the operands are 8- or 11-bit-mantissa values); the mean is rounded
// once to fp32.
// ------------------------------------------------------------------------------------------------
struct PoolParams {
    const void* x[2];
    int64_t stride[2][3];  // elements
    float* pooled[2];      // each [batch][heads][blocks][dim]
    int heads, dim, dtype;
    int img_blocks, blocks;
    Grid g;
};

// Eight consecutive channels of one token: loaded raw (so that several loads can be in flight in
// few registers) and widened to fp32 where they are consumed.
template <typename T>
struct Raw8 {
    uint4 v;
    __device__ __forceinline__ void load(const T* ptr) { v = *reinterpret_cast<const uint4*>(ptr); }
    __device__ __forceinline__ void zero() { v = make_uint4(0, 0, 0, 0); }
    __device__ __forceinline__ void widen(float (&out)[8]) const;
};
template <>
__device__ __forceinline__ void Raw8<__nv_bfloat16>::widen(float (&out)[8]) const {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        out[2 * i] = __uint_as_float(w[i] << 16);
        out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
template <>
__device__ __forceinline__ void Raw8<__half>::widen(float (&out)[8]) const {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        out[2 * i] = f.x;
        out[2 * i + 1] = f.y;
    }
}
template <>
struct Raw8<float> {
    float4 a, b;
    __device__ __forceinline__ void load(const float* ptr) {
        a = *reinterpret_cast<const float4*>(ptr);
        b = *reinterpret_cast<const float4*>(ptr + 4);
    }
    __device__ __forceinline__ void zero() { a = b = make_float4(0, 0, 0, 0); }
    __device__ __forceinline__ void widen(float (&out)[8]) const {
        out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
        out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
    }
};

template <typename T>
__global__ void __launch_bounds__(256) rf_pool_kernel(const PoolParams p, int ntensors) {
    extern __shared__ double red[];  // [row groups][dim]
    __shared__ int src_tok[128];     // source token of each position of the block
    const int blk = blockIdx.x, head = blockIdx.y;
    const int which = ntensors == 2 ? (blockIdx.z & 1) : 0;
    const int batch = ntensors == 2 ? (blockIdx.z >> 1) : blockIdx.z;
    const int lanes = p.dim >> 3;           // threads per token row
    const int groups = 256 / lanes;         // token rows in flight
    const int c = threadIdx.x % lanes, grp = threadIdx.x / lanes;

    int first, count;
    if (blk < p.img_blocks) {
        first = blk * 128;
        count = min(128, p.g.img - first);
    } else {
        first = p.g.img + (blk - p.img_blocks) * 128;
        count = min(128, p.g.img + p.g.txt - first);
    }
    // The permutation's index arithmetic (several integer divisions) once per row, not per lane.
    if (threadIdx.x < count) src_tok[threadIdx.x] = source_of(p.g, first + threadIdx.x);
    __syncthreads();
    const T* base = static_cast<const T*>(p.x[which]) + batch * p.stride[which][0] + head * p.stride[which][1] + c * 8;
    const int64_t tok_stride = p.stride[which][2];
    double acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (grp < groups) {
        // Eight rows per trip: the loads are issued back to back before any of them is consumed.
        for (int r = grp; r < count; r += 8 * groups) {
            Raw8<T> raw[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int rr = r + u * groups;
                if (rr < count) raw[u].load(base + src_tok[rr] * tok_stride);
                else raw[u].zero();
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                float vals[8];
                raw[u].widen(vals);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] += static_cast<double>(vals[i]);
            }
        }
        // Channel c*8+i of row group grp goes to [grp][i][c]: consecutive lanes, consecutive slots.
#pragma unroll
        for (int i = 0; i < 8; ++i) red[grp * p.dim + i * lanes + c] = acc[i];
    }
    __syncthreads();
    for (int ch = threadIdx.x; ch < p.dim; ch += 256) {
        double s = 0;
        const int slot = (ch & 7) * lanes + (ch >> 3);
        for (int g2 = 0; g2 < groups; ++g2) s += red[g2 * p.dim + slot];
        const int64_t o = ((static_cast<int64_t>(batch) * p.heads + head) * p.blocks + blk) * p.dim + ch;
        p.pooled[which][o] = static_cast<float>(s / static_cast<double>(count));
    }
}

// ------------------------------------------------------------------------------------------------
// Scores, threshold, mask.  One CTA per (group of `rows` q-blocks, head, batch); 256 threads.
// Scores are fp64 dot products of the fp32 pooled means; the softmax of the reference is a
// monotone map of each row, so the k-th largest is selected on the raw scores.
// ------------------------------------------------------------------------------------------------
struct MaskParams {
    const float* q_pooled;  // [batch][heads][blocks][dim]
    const float* k_pooled;
    int heads, dim, blocks;
    int vec_shift;  // log2(dim / 4)
    int keep_len;
    int txt_blocks, first_frame_blocks;
    int band;  // < 0: off
    Grid g;
    int img_blocks;
    int8_t* mask;         // [batch][heads][blocks][blocks]
    int64_t* select_idx;  // [blocks][heads][blocks], batch 0
    int64_t* select_num;  // [blocks][heads]
};

__device__ __forceinline__ unsigned long long order_key(double v) {
    const unsigned long long b = static_cast<unsigned long long>(__double_as_longlong(v));
    return (b >> 63) ? ~b : (b | 0x8000000000000000ull);
}

constexpr int kMaskRows = 8;    // q blocks per CTA = M of the fp64 tensor-core tile
constexpr int kMaskTile = 64;   // k blocks staged per trip: eight per warp

__device__ __forceinline__ void dmma884(double& c0, double& c1, double a, double b) {
    asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0, %1}, {%2}, {%3}, {%0, %1};"
                 : "+d"(c0), "+d"(c1)
                 : "d"(a), "d"(b));
}

// kKeysPerLane: ceil(blocks / 32) rounded up to a supported size; the row's keys live in registers
// during the threshold search.
template <int kKeysPerLane>
__global__ void __launch_bounds__(256) rf_mask_kernel(const MaskParams p) {
    extern __shared__ unsigned char smem_dyn[];
    // layout: q rows [8][dim + 4] fp64 | keys [8][blocks] u64 | k tile [64][dim + 4] fp32.
    // q is widened to fp64 once; k is staged as it lies (fp32) and widened in the fragment load.  The
    // pitch dim + 4 makes both fragment loads (8 rows x 4 consecutive channels) conflict-free.
    const int pitch = p.dim + 4;
    double* sq = reinterpret_cast<double*>(smem_dyn);
    unsigned long long* keys = reinterpret_cast<unsigned long long*>(sq + kMaskRows * pitch);
    float* sk = reinterpret_cast<float*>(keys + static_cast<size_t>(kMaskRows) * p.blocks);

    const int row0 = blockIdx.x * kMaskRows, head = blockIdx.y, batch = blockIdx.z;
    const int nrows = min(kMaskRows, p.blocks - row0);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const float* qp = p.q_pooled + ((static_cast<int64_t>(batch) * p.heads + head) * p.blocks) * p.dim;
    const float* kp = p.k_pooled + ((static_cast<int64_t>(batch) * p.heads + head) * p.blocks) * p.dim;

    // Staging: dim is a power of two; a thread moves 4 consecutive channels (one 16-byte load).
    const int vec_per_row = p.dim >> 2, vshift = p.vec_shift;  // vec_per_row == 1 << vshift
    for (int i = tid; i < kMaskRows * vec_per_row; i += 256) {
        const int r = i >> vshift, v = i & (vec_per_row - 1);
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < nrows) x = *reinterpret_cast<const float4*>(qp + static_cast<int64_t>(row0 + r) * p.dim + v * 4);
        double2* d = reinterpret_cast<double2*>(sq + r * pitch + v * 4);
        d[0] = make_double2(static_cast<double>(x.x), static_cast<double>(x.y));
        d[1] = make_double2(static_cast<double>(x.z), static_cast<double>(x.w));
    }

    // Scores on the fp64 tensor cores: warp w owns k columns 8w..8w+7 of the tile over all channels,
    // as four independent accumulator chains (consecutive MMAs of one chain wait on each other).
    const int frag_row = lane >> 2, frag_k = lane & 3;
    for (int j0 = 0; j0 < p.blocks; j0 += kMaskTile) {
        __syncthreads();
        const int nj = min(kMaskTile, p.blocks - j0);
        for (int i = tid; i < kMaskTile * vec_per_row; i += 256) {
            const int r = i >> vshift, v = i & (vec_per_row - 1);
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (r < nj) x = *reinterpret_cast<const float4*>(kp + static_cast<int64_t>(j0 + r) * p.dim + v * 4);
            *reinterpret_cast<float4*>(sk + r * pitch + v * 4) = x;
        }
        __syncthreads();
        double c[4][2] = {{0.0, 0.0}, {0.0, 0.0}, {0.0, 0.0}, {0.0, 0.0}};
        const double* a_ptr = sq + frag_row * pitch + frag_k;
        const float* b_ptr = sk + (warp * 8 + frag_row) * pitch + frag_k;
        int ch = 0;
        for (; ch + 16 <= p.dim; ch += 16) {
#pragma unroll
            for (int u = 0; u < 4; ++u)
                dmma884(c[u][0], c[u][1], a_ptr[ch + 4 * u], static_cast<double>(b_ptr[ch + 4 * u]));
        }
        for (; ch < p.dim; ch += 4) dmma884(c[0][0], c[0][1], a_ptr[ch], static_cast<double>(b_ptr[ch]));
        const double s0 = (c[0][0] + c[1][0]) + (c[2][0] + c[3][0]);
        const double s1 = (c[0][1] + c[1][1]) + (c[2][1] + c[3][1]);
        const int col = j0 + warp * 8 + frag_k * 2;
        if (frag_row < nrows) {
            if (col < p.blocks) keys[static_cast<size_t>(frag_row) * p.blocks + col] = order_key(s0);
            if (col + 1 < p.blocks) keys[static_cast<size_t>(frag_row) * p.blocks + col + 1] = order_key(s1);
        }
    }
    __syncthreads();

    // One warp per row.  Bitwise search for the largest key value that at least keep_len keys reach;
    // a key of 0 (padding) never counts because every candidate is at least 1.
    for (int r = warp; r < nrows; r += 8) {
        const unsigned long long* kr = keys + static_cast<size_t>(r) * p.blocks;
        unsigned long long mine[kKeysPerLane];
#pragma unroll
        for (int i = 0; i < kKeysPerLane; ++i) {
            const int j = lane + 32 * i;
            mine[i] = j < p.blocks ? kr[j] : 0ull;
        }
        // High words first (32 steps on 32-bit compares); the low words only matter among the keys that
        // share the threshold's high word, which is almost always a single key.
        unsigned int thr_hi = 0;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned int cand = thr_hi | (1u << bit);
            int cnt = 0;
#pragma unroll
            for (int i = 0; i < kKeysPerLane; ++i) cnt += static_cast<unsigned int>(mine[i] >> 32) >= cand;
            cnt = __reduce_add_sync(0xffffffffu, cnt);
            if (cnt >= p.keep_len) thr_hi = cand;
        }
        int above = 0, equal = 0;
#pragma unroll
        for (int i = 0; i < kKeysPerLane; ++i) {
            const unsigned int hi = static_cast<unsigned int>(mine[i] >> 32);
            above += hi > thr_hi;
            equal += hi == thr_hi;
        }
        above = __reduce_add_sync(0xffffffffu, above);
        equal = __reduce_add_sync(0xffffffffu, equal);
        unsigned int thr_lo = 0;
        if (equal == 1) {
            unsigned int lo = 0;
#pragma unroll
            for (int i = 0; i < kKeysPerLane; ++i)
                if (static_cast<unsigned int>(mine[i] >> 32) == thr_hi) lo = static_cast<unsigned int>(mine[i]);
            thr_lo = __reduce_or_sync(0xffffffffu, lo);
        } else {
            const int want = p.keep_len - above;  // rank of the threshold among the keys that tie on the high word
            for (int bit = 31; bit >= 0; --bit) {
                const unsigned int cand = thr_lo | (1u << bit);
                int cnt = 0;
#pragma unroll
                for (int i = 0; i < kKeysPerLane; ++i)
                    cnt += static_cast<unsigned int>(mine[i] >> 32) == thr_hi && static_cast<unsigned int>(mine[i]) >= cand;
                cnt = __reduce_add_sync(0xffffffffu, cnt);
                if (cnt >= want) thr_lo = cand;
            }
        }
        const unsigned long long thr = (static_cast<unsigned long long>(thr_hi) << 32) | thr_lo;
        const int qb = row0 + r;
        const bool row_forced = qb >= p.blocks - p.txt_blocks || qb < p.first_frame_blocks;
        // Frame range of the q block (image blocks only), for the optional temporal band.
        int q_lo = 0, q_hi = 0;
        const bool q_img = qb < p.img_blocks;
        if (p.band >= 0 && q_img) {
            q_lo = (qb * 128) / p.g.hw;
            q_hi = (min(qb * 128 + 128, p.g.img) - 1) / p.g.hw;
        }
        int8_t* mrow = p.mask ? p.mask + ((static_cast<int64_t>(batch) * p.heads + head) * p.blocks + qb) * p.blocks : nullptr;
        int64_t* lrow = (p.select_idx && batch == 0)
                            ? p.select_idx + (static_cast<int64_t>(qb) * p.heads + head) * p.blocks
                            : nullptr;
        int kept = 0;
#pragma unroll
        for (int i = 0; i < kKeysPerLane; ++i) {
            const int j = lane + 32 * i;
            if (32 * i >= p.blocks) break;  // warp-uniform
            bool keep = false;
            if (j < p.blocks) {
                keep = row_forced || mine[i] >= thr || j >= p.blocks - p.txt_blocks || j < p.first_frame_blocks;
                if (!keep && p.band >= 0 && q_img && j < p.img_blocks) {
                    const int k_lo = (j * 128) / p.g.hw;
                    const int k_hi = (min(j * 128 + 128, p.g.img) - 1) / p.g.hw;
                    keep = (k_lo - p.band <= q_hi) && (q_lo - p.band <= k_hi);
                }
                if (mrow) mrow[j] = keep ? 1 : 0;
            }
            const unsigned ballot = __ballot_sync(0xffffffffu, keep);
            if (lrow && keep) lrow[kept + __popc(ballot & ((1u << lane) - 1u))] = j;
            kept += __popc(ballot);
        }
        if (lrow) {
            for (int j = kept + lane; j < p.blocks; j += 32) lrow[j] = -1;
            if (lane == 0 && p.select_num) p.select_num[static_cast<int64_t>(qb) * p.heads + head] = kept;
        }
    }
}

size_t mask_smem_bytes(int dim, int blocks) {
    return (static_cast<size_t>(kMaskRows) * (dim + 4) + static_cast<size_t>(kMaskRows) * blocks) * 8 +
           static_cast<size_t>(kMaskTile) * (dim + 4) * 4;
}

}  // namespace

}  // namespace sdb

using namespace sdb;

extern "C" int mindiesd_rf_rearrange(const mindiesd_rearrange_args* a, void* stream) {
    if (!a || !a->src || !a->dst) return MINDIESD_E_NULL;
    if (a->src == a->dst) return MINDIESD_E_VALUE;
    if (a->batch <= 0 || a->heads <= 0 || a->seq <= 0 || a->head_dim <= 0) return MINDIESD_E_SHAPE;
    const int eb = a->elem_bytes;
    if (eb != 1 && eb != 2 && eb != 4) return MINDIESD_E_DTYPE;
    const int vec = 16 / eb;  // elements per 16-byte vector
    if (a->head_dim % vec || a->head_dim / vec > 256) return MINDIESD_E_SHAPE;
    if (a->t <= 0 || a->h <= 0 || a->w <= 0 || a->txt_len < 0) return MINDIESD_E_SHAPE;
    if (static_cast<int64_t>(a->t) * a->h * a->w + a->txt_len != a->seq) return MINDIESD_E_SHAPE;
    // The reference's permutation is undefined for a ragged grid with fewer than 8 rows or columns.
    if ((a->h % 8 || a->w % 8) && (a->h < 8 || a->w < 8)) return MINDIESD_E_SHAPE;
    if (static_cast<int64_t>(a->batch) * a->heads > 65535) return MINDIESD_E_SHAPE;
    if (reinterpret_cast<uintptr_t>(a->src) % 16 || reinterpret_cast<uintptr_t>(a->dst) % 16) return MINDIESD_E_STRIDE;
    RearrangeParams p;
    p.src = static_cast<const uint4*>(a->src);
    p.dst = static_cast<uint4*>(a->dst);
    for (int i = 0; i < 3; ++i) {
        if (a->src_stride[i] % vec || a->dst_stride[i] % vec) return MINDIESD_E_STRIDE;
        p.src_stride[i] = a->src_stride[i] / vec;
        p.dst_stride[i] = a->dst_stride[i] / vec;
    }
    p.heads = a->heads;
    p.seq = a->seq;
    p.vec_per_row = a->head_dim / vec;
    p.g = make_grid(a->t, a->h, a->w, a->txt_len);
    p.inverse = a->inverse ? 1 : 0;
    dim3 grid((a->seq + kRearrangeRows - 1) / kRearrangeRows, a->batch * a->heads);
    rf_rearrange_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? MINDIESD_OK : static_cast<int>(e);
}

extern "C" size_t mindiesd_rf_block_mask_scratch_bytes(int32_t batch, int32_t heads, int32_t seq, int32_t head_dim) {
    if (batch <= 0 || heads <= 0 || seq <= 0 || head_dim <= 0) return 0;
    // Image and text are pooled separately, so there is at most one block more than ceil(seq / 128).
    const size_t blocks = static_cast<size_t>(seq + 127) / 128 + 1;
    return static_cast<size_t>(batch) * 2 * heads * blocks * head_dim * sizeof(float);
}

namespace sdb {

namespace {

bool grid_ok(int t, int h, int w, int txt_len, int64_t seq) {
    if (t < 0 || h < 0 || w < 0 || txt_len < 0) return false;
    if (static_cast<int64_t>(t) * h * w + txt_len != seq) return false;
    // The reference's permutation is undefined for a ragged grid with fewer than 8 rows or columns.
    if (static_cast<int64_t>(t) * h * w > 0 && (h % 8 || w % 8) && (h < 8 || w < 8)) return false;
    return true;
}

int launch_pool(const void* const x[2], const int64_t* const stride[2], float* const pooled[2], int ntensors, int batch,
                int heads, int seq, int dim, int dtype, const Grid& g, cudaStream_t stream) {
    if (dim <= 0 || dim % 8 || dim > 256 || 256 % (dim / 8)) return MINDIESD_E_SHAPE;
    if (dtype != MINDIESD_BF16 && dtype != MINDIESD_FP16 && dtype != MINDIESD_FP32) return MINDIESD_E_DTYPE;
    if (batch <= 0 || heads <= 0 || seq <= 0 || batch > 32767 || heads > 65535) return MINDIESD_E_SHAPE;
    const int vec = 16 / dtype_bytes(dtype);
    PoolParams pp;
    for (int w = 0; w < 2; ++w) {
        const int src = w < ntensors ? w : 0;
        if (!x[src] || !pooled[src]) return MINDIESD_E_NULL;
        if (reinterpret_cast<uintptr_t>(x[src]) % 16 || reinterpret_cast<uintptr_t>(pooled[src]) % 4) return MINDIESD_E_STRIDE;
        pp.x[w] = x[src];
        pp.pooled[w] = pooled[src];
        for (int i = 0; i < 3; ++i) {
            if (stride[src][i] % vec) return MINDIESD_E_STRIDE;
            pp.stride[w][i] = stride[src][i];
        }
    }
    pp.heads = heads;
    pp.dim = dim;
    pp.dtype = dtype;
    pp.img_blocks = (g.img + 127) / 128;
    pp.blocks = pp.img_blocks + (g.txt + 127) / 128;
    pp.g = g;
    dim3 grid(pp.blocks, heads, batch * ntensors);
    const size_t smem = static_cast<size_t>(256 / (dim / 8)) * dim * sizeof(double);
    if (dtype == MINDIESD_BF16)
        rf_pool_kernel<__nv_bfloat16><<<grid, 256, smem, stream>>>(pp, ntensors);
    else if (dtype == MINDIESD_FP16)
        rf_pool_kernel<__half><<<grid, 256, smem, stream>>>(pp, ntensors);
    else
        rf_pool_kernel<float><<<grid, 256, smem, stream>>>(pp, ntensors);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? MINDIESD_OK : static_cast<int>(e);
}

int launch_mask(const float* q_pooled, const float* k_pooled, int batch, int heads, int dim, const Grid& g,
                double sparsity, int protect_first_frame, int band, int8_t* mask, int64_t* select_idx,
                int64_t* select_num, cudaStream_t stream) {
    if (!q_pooled || !k_pooled) return MINDIESD_E_NULL;
    if (!mask && !select_idx) return MINDIESD_E_NULL;
    if (select_idx && !select_num) return MINDIESD_E_NULL;
    if (batch <= 0 || heads <= 0 || dim <= 0 || batch > 65535 || heads > 65535) return MINDIESD_E_SHAPE;
    if (!(sparsity >= 0.0) || !(sparsity < 1.0)) return MINDIESD_E_VALUE;
    MaskParams mp;
    mp.q_pooled = q_pooled;
    mp.k_pooled = k_pooled;
    mp.heads = heads;
    mp.dim = dim;
    mp.img_blocks = (g.img + 127) / 128;
    mp.txt_blocks = (g.txt + 127) / 128;
    mp.blocks = mp.img_blocks + mp.txt_blocks;
    if (mp.blocks < 1) return MINDIESD_E_SHAPE;
    if (mp.blocks > kMaxMaskBlocks) return MINDIESD_E_CAPACITY;
    // Same double-precision expression as the reference's math.ceil(cols * (1 - sparsity)).
    mp.keep_len = static_cast<int>(ceil(static_cast<double>(mp.blocks) * (1.0 - sparsity)));
    if (mp.keep_len < 1) return MINDIESD_E_VALUE;
    if (mp.keep_len > mp.blocks) mp.keep_len = mp.blocks;
    mp.first_frame_blocks = protect_first_frame ? (g.hw + 127) / 128 : 0;
    if (mp.first_frame_blocks > mp.blocks) mp.first_frame_blocks = mp.blocks;
    mp.band = band;
    mp.g = g;
    mp.mask = mask;
    mp.select_idx = select_idx;
    mp.select_num = select_num;
    if (dim < 16 || dim > 512 || (dim & (dim - 1))) return MINDIESD_E_SHAPE;  // power of two
    mp.vec_shift = 0;
    while ((4 << mp.vec_shift) < dim) ++mp.vec_shift;
    if (reinterpret_cast<uintptr_t>(q_pooled) % 16 || reinterpret_cast<uintptr_t>(k_pooled) % 16) return MINDIESD_E_STRIDE;
    const size_t smem = mask_smem_bytes(mp.dim, mp.blocks);
    dim3 grid((mp.blocks + kMaskRows - 1) / kMaskRows, heads, batch);
    auto launch = [&](auto kernel) -> cudaError_t {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return e;
        kernel<<<grid, 256, smem, stream>>>(mp);
        return cudaGetLastError();
    };
    const int per_lane = (mp.blocks + 31) / 32;
    cudaError_t e;
    if (per_lane <= 8) e = launch(rf_mask_kernel<8>);
    else if (per_lane <= 20) e = launch(rf_mask_kernel<20>);
    else if (per_lane <= 32) e = launch(rf_mask_kernel<32>);
    else e = launch(rf_mask_kernel<64>);
    return e == cudaSuccess ? MINDIESD_OK : static_cast<int>(e);
}

}  // namespace

int rf_block_mask_impl(const mindiesd_mask_args* a, float* pooled, size_t pooled_bytes, cudaStream_t stream) {
    if (!a || !a->q || !a->k || !pooled) return MINDIESD_E_NULL;
    if (a->block_size != 128) return MINDIESD_E_SHAPE;
    if (a->batch <= 0 || a->heads <= 0 || a->seq <= 0 || a->head_dim <= 0) return MINDIESD_E_SHAPE;
    if (a->t <= 0 || a->h <= 0 || a->w <= 0) return MINDIESD_E_SHAPE;
    if (!grid_ok(a->t, a->h, a->w, a->txt_len, a->seq)) return MINDIESD_E_SHAPE;
    if (!(a->scale > 0.0f)) return MINDIESD_E_VALUE;
    const Grid g = make_grid(a->t, a->h, a->w, a->txt_len);
    const int blocks = (g.img + 127) / 128 + (a->txt_len + 127) / 128;
    const size_t per_tensor = static_cast<size_t>(a->batch) * a->heads * blocks * a->head_dim;
    if (pooled_bytes < 2 * per_tensor * sizeof(float)) return MINDIESD_E_CAPACITY;
    if (reinterpret_cast<uintptr_t>(pooled) % 16) return MINDIESD_E_STRIDE;
    const void* x[2] = {a->q, a->k};
    const int64_t* strides[2] = {a->q_stride, a->k_stride};
    float* out[2] = {pooled, pooled + per_tensor};
    int rc = launch_pool(x, strides, out, 2, a->batch, a->heads, a->seq, a->head_dim, a->dtype, g, stream);
    if (rc) return rc;
    return launch_mask(out[0], out[1], a->batch, a->heads, a->head_dim, g, a->sparsity, a->protect_first_frame,
                       a->temporal_band, a->mask, a->select_idx, a->select_num, stream);
}
}  // namespace sdb

extern "C" int mindiesd_rf_block_mask(const mindiesd_mask_args* a, void* stream) {
    if (!a) return MINDIESD_E_NULL;
    return rf_block_mask_impl(a, static_cast<float*>(a->scratch), a->scratch_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int mindiesd_rf_pool(const mindiesd_pool_args* a, void* stream) {
    if (!a || !a->x || !a->pooled) return MINDIESD_E_NULL;
    if (a->block_size != 128) return MINDIESD_E_SHAPE;
    Grid g;
    if (a->permute) {
        if (a->t <= 0 || a->h <= 0 || a->w <= 0) return MINDIESD_E_SHAPE;
        if (!grid_ok(a->t, a->h, a->w, a->txt_len, a->seq)) return MINDIESD_E_SHAPE;
        g = make_grid(a->t, a->h, a->w, a->txt_len);
    } else {
        g = make_grid(0, 1, 1, a->seq);  // no image part: consecutive tokens are pooled as they lie
    }
    const void* x[2] = {a->x, a->x};
    const int64_t* strides[2] = {a->x_stride, a->x_stride};
    float* out[2] = {a->pooled, a->pooled};
    return launch_pool(x, strides, out, 1, a->batch, a->heads, a->seq, a->head_dim, a->dtype, g,
                       static_cast<cudaStream_t>(stream));
}

extern "C" int mindiesd_rf_mask_from_pooled(const mindiesd_pooled_mask_args* a, void* stream) {
    if (!a) return MINDIESD_E_NULL;
    if (a->block_size != 128) return MINDIESD_E_SHAPE;
    if (a->t <= 0 || a->h <= 0 || a->w <= 0 || a->txt_len < 0) return MINDIESD_E_SHAPE;
    const Grid g = make_grid(a->t, a->h, a->w, a->txt_len);
    const int blocks = (g.img + 127) / 128 + (a->txt_len + 127) / 128;
    if (blocks != a->blocks) return MINDIESD_E_SHAPE;
    if (a->head_dim > 1024) return MINDIESD_E_SHAPE;
    return launch_mask(a->q_pooled, a->k_pooled, a->batch, a->heads, a->head_dim, g, a->sparsity,
                       a->protect_first_frame, a->temporal_band, a->mask, a->select_idx, a->select_num,
                       static_cast<cudaStream_t>(stream));
}

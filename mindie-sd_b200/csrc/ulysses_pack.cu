// Data movement around sequence-parallel (Ulysses) attention, and rotary position embedding.
//
// ulysses_move_kernel   this rank's [rows, N, 128] slices of q, k, v  ->  per destination rank a
//                       [rows, n_src * heads, 128] block holding the heads that rank owns (forward),
//                       optionally rotating q and k by the rotary embedding on the way; or the inverse:
//                       per source rank a [rows, heads, 128] block -> this rank's [rows, N, 128] output.
//                       The per-rank side is a table of pointers, so the same kernel fills a local
//                       send buffer (one chunk per destination) or stores straight into the receive
//                       buffers of the peers over NVLink.
// rope_kernel           rotary position embedding of a 4-D tensor, half or interleaved rotation.
//
// Both are pure data movement: 16-byte vectors, several loads in flight per thread, HBM/NVLink bound.
#include "capi_common.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace sdb {

namespace {

constexpr int kVec = 8;  // 2-byte elements per 16-byte vector

struct MoveParams {
    const uint8_t* tensor[3];   // the [rows, N, 128] side (q, k, v or the output)
    uint8_t* table[MINDIESD_MAX_RANKS];  // the per-rank side
    int64_t tensor_row_stride, tensor_head_stride;  // elements
    int64_t table_row_stride;                       // elements
    int n_src, rows, world, group_heads, head0, heads;
    int inverse;
    const float* cos;
    const float* sin;
    int rope_mode;  // 0 none, 1 half, 2 interleaved
};

template <typename T>
struct Pair;
template <>
struct Pair<__nv_bfloat16> {
    using type = __nv_bfloat162;
    static __device__ __forceinline__ float2 up(type v) { return __bfloat1622float2(v); }
    static __device__ __forceinline__ type down(float a, float b) { return __floats2bfloat162_rn(a, b); }
};
template <>
struct Pair<__half> {
    using type = __half2;
    static __device__ __forceinline__ float2 up(type v) { return __half22float2(v); }
    static __device__ __forceinline__ type down(float a, float b) { return __floats2half2_rn(a, b); }
};

// Rotary embedding of one 8-channel vector in fp32, the arithmetic of the reference's unfused branch
// (mindiesd/layers/rope.py:104-113 of MindIE-SD): x * cos + rotated(x) * sin with both products rounded
// before the sum, one rounding to the element type at the end.
//   interleaved: rotated(x) = (-x1, x0, -x3, x2, ...): the partner sits in the same vector
//   half:        rotated(x) = (-x[d/2:], x[:d/2]): the partner vector is d/2 channels away (`other`)
template <typename T>
__device__ __forceinline__ uint4 rope_vec(uint4 own, uint4 other, const float* cos, const float* sin, int mode,
                                          bool upper_half) {
    using P = Pair<T>;
    const typename P::type* xo = reinterpret_cast<const typename P::type*>(&own);
    const typename P::type* xp = reinterpret_cast<const typename P::type*>(&other);
    const float4 c0 = reinterpret_cast<const float4*>(cos)[0], c1 = reinterpret_cast<const float4*>(cos)[1];
    const float4 s0 = reinterpret_cast<const float4*>(sin)[0], s1 = reinterpret_cast<const float4*>(sin)[1];
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    uint4 out;
    typename P::type* o = reinterpret_cast<typename P::type*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 x = P::up(xo[i]);
        float r0, r1;
        if (mode == 2) {
            r0 = -x.y;
            r1 = x.x;
        } else {
            const float2 y = P::up(xp[i]);
            r0 = upper_half ? y.x : -y.x;
            r1 = upper_half ? y.y : -y.y;
        }
        o[i] = P::down(__fadd_rn(__fmul_rn(x.x, c[2 * i]), __fmul_rn(r0, s[2 * i])),
                       __fadd_rn(__fmul_rn(x.y, c[2 * i + 1]), __fmul_rn(r1, s[2 * i + 1])));
    }
    return out;
}

// One work item = one 16-byte vector.  Within a token row the items are numbered so that consecutive
// threads touch consecutive addresses on both sides: vector within a head (16), head of the piece, tensor
// (q, k, v), rank.  What a thread moves is the same in every row, so its item numbers are taken apart once
// (the divisions by run-time values cost more than the copy) and the loop over the thread block's rows only
// adds the row strides; two rows are in flight per pass when nothing is rotated.
template <typename T, bool kRotate>
__global__ void __launch_bounds__(256, 2) ulysses_move_kernel(const MoveParams p) {
    constexpr int kVecsPerHead = 128 / kVec;  // 16
    constexpr int kItems = 4;                 // items of one row a thread holds at a time
    constexpr int kRows = kRotate ? 1 : 2;    // rows in flight per pass
    const int per_tensor = p.heads * kVecsPerHead;
    const int per_rank = p.n_src * per_tensor;
    const int per_row = per_rank * p.world;
    const int64_t t_stride = p.tensor_row_stride * 2, b_stride = p.table_row_stride * 2;  // bytes per row
    const int64_t src_stride = p.inverse ? b_stride : t_stride, dst_stride = p.inverse ? t_stride : b_stride;
    for (int base = threadIdx.x; base < per_row; base += blockDim.x * kItems) {
        const uint8_t* src[kItems];
        uint8_t* dst[kItems];
        int vec_of[kItems];  // vector index within the head if the item is rotated, else -1
        bool on[kItems];
#pragma unroll
        for (int u = 0; u < kItems; ++u) {
            const int item = base + u * blockDim.x;
            on[u] = item < per_row;
            const int it = on[u] ? item : 0;
            const int rank = it / per_rank;
            int r = it - rank * per_rank;
            const int which = r / per_tensor;
            r -= which * per_tensor;
            const int head = r / kVecsPerHead;
            const int vec = r % kVecsPerHead;
            const int64_t t_off = ((rank * p.group_heads + p.head0 + head) * p.tensor_head_stride + vec * kVec) * 2;
            const int64_t b_off = (static_cast<int64_t>(which * p.heads + head) * 128 + vec * kVec) * 2;
            vec_of[u] = (kRotate && which < 2) ? vec : -1;
            if (!p.inverse) {
                src[u] = p.tensor[which] + t_off;
                dst[u] = p.table[rank] + b_off;
            } else {
                src[u] = p.table[rank] + b_off;
                dst[u] = const_cast<uint8_t*>(p.tensor[0]) + t_off;
            }
        }
        for (int row0 = blockIdx.x * kRows; row0 < p.rows; row0 += gridDim.x * kRows) {
            uint4 val[kRows][kItems];
            uint4 partner[kItems];
#pragma unroll
            for (int rr = 0; rr < kRows; ++rr) {
                const int row = row0 + rr;
#pragma unroll
                for (int u = 0; u < kItems; ++u) {
                    if (!on[u] || row >= p.rows) continue;
                    const uint8_t* s_ptr = src[u] + row * src_stride;
                    val[rr][u] = *reinterpret_cast<const uint4*>(s_ptr);
                    if (kRotate && vec_of[u] >= 0 && p.rope_mode == 1)
                        partner[u] = *reinterpret_cast<const uint4*>(s_ptr + ((vec_of[u] < 8) ? 128 : -128));
                }
            }
#pragma unroll
            for (int rr = 0; rr < kRows; ++rr) {
                const int row = row0 + rr;
#pragma unroll
                for (int u = 0; u < kItems; ++u) {
                    if (!on[u] || row >= p.rows) continue;
                    uint4 v = val[rr][u];
                    if (kRotate && vec_of[u] >= 0) {
                        const float* c = p.cos + static_cast<int64_t>(row) * 128 + vec_of[u] * kVec;
                        const float* sn = p.sin + static_cast<int64_t>(row) * 128 + vec_of[u] * kVec;
                        v = rope_vec<T>(v, partner[u], c, sn, p.rope_mode, vec_of[u] >= 8);
                    }
                    *reinterpret_cast<uint4*>(dst[u] + row * dst_stride) = v;
                }
            }
        }
    }
    // The destinations may be another GPU's memory: make this thread's stores visible system-wide before
    // the kernel counts as complete, so that whatever orders the ranks afterwards also orders the data.
    __threadfence_system();
}

struct RopeParams {
    const uint8_t* x;
    uint8_t* out;
    const void* cos;
    const void* sin;
    int64_t x_stride[3], o_stride[3];  // elements: batch, head, token
    int batch, heads, seq, dim;
    int mode;        // 1 half, 2 interleaved
    int table_fp32;  // tables are fp32 (else the element type of x)
};

// Scalar form for any even head dim and any element type: one thread per channel pair.
template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f(float v) { return v; }
template <>
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }

template <typename T>
__global__ void __launch_bounds__(256) rope_kernel(const RopeParams p) {
    const int half = p.dim / 2;
    const int64_t total = static_cast<int64_t>(p.batch) * p.heads * p.seq * half;
    for (int64_t item = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; item < total;
         item += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int pair = static_cast<int>(item % half);
        int64_t r = item / half;
        const int head = static_cast<int>(r % p.heads);
        r /= p.heads;
        const int tok = static_cast<int>(r % p.seq);
        const int b = static_cast<int>(r / p.seq);
        // the two channels this thread produces, and the channels their rotated partners come from
        const int c0 = p.mode == 2 ? 2 * pair : pair;
        const int c1 = p.mode == 2 ? 2 * pair + 1 : pair + half;
        const T* x = reinterpret_cast<const T*>(p.x) + b * p.x_stride[0] + head * p.x_stride[1] + tok * p.x_stride[2];
        T* o = reinterpret_cast<T*>(p.out) + b * p.o_stride[0] + head * p.o_stride[1] + tok * p.o_stride[2];
        const float x0 = to_f(x[c0]), x1 = to_f(x[c1]);
        const int64_t t = static_cast<int64_t>(tok) * p.dim;
        float y0, y1;
        if (p.table_fp32) {
            const float* cs = static_cast<const float*>(p.cos);
            const float* sn = static_cast<const float*>(p.sin);
            y0 = __fadd_rn(__fmul_rn(x0, cs[t + c0]), __fmul_rn(-x1, sn[t + c0]));
            y1 = __fadd_rn(__fmul_rn(x1, cs[t + c1]), __fmul_rn(x0, sn[t + c1]));
        } else {
            // tables in the element type: the reference then multiplies and adds in that type, every
            // intermediate rounded to it
            const T* cs = static_cast<const T*>(p.cos);
            const T* sn = static_cast<const T*>(p.sin);
            auto rnd = [](float v) { return to_f(from_f<T>(v)); };
            y0 = rnd(x0 * to_f(cs[t + c0])) + rnd(-x1 * to_f(sn[t + c0]));
            y1 = rnd(x1 * to_f(cs[t + c1])) + rnd(x0 * to_f(sn[t + c1]));
        }
        o[c0] = from_f<T>(y0);
        o[c1] = from_f<T>(y1);
    }
}

int grid_for(int64_t items, int per_thread, int requested) {
    if (requested > 0) return requested;
    const int64_t blocks = (items + 256LL * per_thread - 1) / (256LL * per_thread);
    const int64_t cap = 148LL * 8;
    return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace
}  // namespace sdb

using namespace sdb;

extern "C" int mindiesd_ulysses_move(const mindiesd_ulysses_move_args* a, void* stream) {
    if (!a) return MINDIESD_E_NULL;
    if (a->head_dim != 128) return MINDIESD_E_SHAPE;
    if (a->dtype != MINDIESD_BF16 && a->dtype != MINDIESD_FP16) return MINDIESD_E_DTYPE;
    if (a->world < 1 || a->world > MINDIESD_MAX_RANKS || a->rows <= 0 || a->heads <= 0 || a->group_heads <= 0 ||
        a->head0 < 0 || a->head0 + a->heads > a->group_heads)
        return MINDIESD_E_SHAPE;
    const int n_src = a->inverse ? 1 : a->n_src;
    if (n_src < 1 || n_src > 3) return MINDIESD_E_SHAPE;
    if (a->rope_mode < 0 || a->rope_mode > 2) return MINDIESD_E_VALUE;
    if (a->rope_mode != 0 && (a->inverse || !a->cos || !a->sin)) return a->inverse ? MINDIESD_E_VALUE : MINDIESD_E_NULL;
    MoveParams p = {};
    for (int i = 0; i < n_src; ++i) {
        if (!a->tensor[i]) return MINDIESD_E_NULL;
        if (reinterpret_cast<uintptr_t>(a->tensor[i]) % 16) return MINDIESD_E_STRIDE;
        p.tensor[i] = static_cast<const uint8_t*>(a->tensor[i]);
    }
    for (int r = 0; r < a->world; ++r) {
        if (!a->table[r]) return MINDIESD_E_NULL;
        if (reinterpret_cast<uintptr_t>(a->table[r]) % 16) return MINDIESD_E_STRIDE;
        p.table[r] = static_cast<uint8_t*>(a->table[r]);
    }
    if (a->tensor_row_stride % kVec || a->tensor_head_stride % kVec || a->table_row_stride % kVec ||
        a->tensor_row_stride < 0 || a->tensor_head_stride < 0 || a->table_row_stride < 0)
        return MINDIESD_E_STRIDE;
    if (a->rope_mode && (reinterpret_cast<uintptr_t>(a->cos) % 16 || reinterpret_cast<uintptr_t>(a->sin) % 16))
        return MINDIESD_E_STRIDE;
    p.tensor_row_stride = a->tensor_row_stride;
    p.tensor_head_stride = a->tensor_head_stride;
    p.table_row_stride = a->table_row_stride;
    p.n_src = n_src;
    p.rows = a->rows;
    p.world = a->world;
    p.group_heads = a->group_heads;
    p.head0 = a->head0;
    p.heads = a->heads;
    p.inverse = a->inverse != 0;
    p.cos = a->cos;
    p.sin = a->sin;
    p.rope_mode = a->rope_mode;
    // One thread block per pass of rows until every SM holds its two; more rows than that are walked in a loop.
    const int rows_per_pass = a->rope_mode ? 1 : 2;
    const int passes = (a->rows + rows_per_pass - 1) / rows_per_pass;
    const int resident = 148 * 2;
    const int grid = a->thread_blocks > 0 ? a->thread_blocks : (passes < resident ? passes : resident);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool bf16 = a->dtype == MINDIESD_BF16;
    if (a->rope_mode) {
        if (bf16) ulysses_move_kernel<__nv_bfloat16, true><<<grid, 256, 0, s>>>(p);
        else ulysses_move_kernel<__half, true><<<grid, 256, 0, s>>>(p);
    } else {
        if (bf16) ulysses_move_kernel<__nv_bfloat16, false><<<grid, 256, 0, s>>>(p);
        else ulysses_move_kernel<__half, false><<<grid, 256, 0, s>>>(p);
    }
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? MINDIESD_OK : static_cast<int>(e);
}

extern "C" int mindiesd_rope(const mindiesd_rope_args* a, void* stream) {
    if (!a || !a->x || !a->out || !a->cos || !a->sin) return MINDIESD_E_NULL;
    if (a->batch <= 0 || a->heads <= 0 || a->seq <= 0 || a->head_dim <= 0 || a->head_dim % 2) return MINDIESD_E_SHAPE;
    if (a->mode != 1 && a->mode != 2) return MINDIESD_E_VALUE;
    if (a->dtype != MINDIESD_BF16 && a->dtype != MINDIESD_FP16 && a->dtype != MINDIESD_FP32) return MINDIESD_E_DTYPE;
    if (a->table_dtype != MINDIESD_FP32 && a->table_dtype != a->dtype) return MINDIESD_E_DTYPE;
    RopeParams p = {};
    p.x = static_cast<const uint8_t*>(a->x);
    p.out = static_cast<uint8_t*>(a->out);
    p.cos = a->cos;
    p.sin = a->sin;
    for (int i = 0; i < 3; ++i) {
        if (a->x_stride[i] < 0 || a->out_stride[i] < 0) return MINDIESD_E_STRIDE;
        p.x_stride[i] = a->x_stride[i];
        p.o_stride[i] = a->out_stride[i];
    }
    p.batch = a->batch;
    p.heads = a->heads;
    p.seq = a->seq;
    p.dim = a->head_dim;
    p.mode = a->mode;
    p.table_fp32 = a->table_dtype == MINDIESD_FP32;
    const int64_t items = static_cast<int64_t>(a->batch) * a->heads * a->seq * (a->head_dim / 2);
    const int grid = grid_for(items, 4, 0);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (a->dtype) {
        case MINDIESD_BF16: rope_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(p); break;
        case MINDIESD_FP16: rope_kernel<__half><<<grid, 256, 0, s>>>(p); break;
        default: rope_kernel<float><<<grid, 256, 0, s>>>(p); break;
    }
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? MINDIESD_OK : static_cast<int>(e);
}

extern "C" int mindiesd_copy_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes,
                                size_t height, void* stream) {
    if (!dst || !src) return MINDIESD_E_NULL;
    if (width_bytes == 0 || height == 0) return MINDIESD_OK;
    if (width_bytes > dst_pitch || width_bytes > src_pitch) return MINDIESD_E_STRIDE;
    const cudaError_t e = cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, height, cudaMemcpyDefault,
                                            static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? MINDIESD_OK : static_cast<int>(e);
}

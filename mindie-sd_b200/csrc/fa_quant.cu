// Dynamic quantisation of attention operands to e4m3 (HBM-bound byte work).
//   mode 0: one scale per (row_block tokens x 128 channels) block;
//   mode 1: one scale per channel over the whole sequence of a (batch, head).
// scale = absmax / 448 (448 = largest finite e4m3), 1 for an all-zero group; stored = x / scale.
#include "capi_common.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace sdb {
namespace {

constexpr float kE4m3Max = 448.0f;

struct QuantParams {
    const void* x;
    uint8_t* out;
    float* scales;
    int64_t stride[3];  // elements
    int heads, seq, row_block, blocks;
    int is_bf16;
};

__device__ __forceinline__ void unpack8(const uint4& raw, int is_bf16, float (&f)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    if (is_bf16) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            f[2 * i] = v.x;
            f[2 * i + 1] = v.y;
        }
    }
}

__device__ __forceinline__ uint2 quant8(const float (&f)[8], float inv) {
    uint16_t h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(h[i]) : "f"(f[2 * i + 1] * inv), "f"(f[2 * i] * inv));
    return make_uint2(static_cast<uint32_t>(h[0]) | (static_cast<uint32_t>(h[1]) << 16),
                      static_cast<uint32_t>(h[2]) | (static_cast<uint32_t>(h[3]) << 16));
}

// mode 0 without rotation.  Grid (row block, head, batch); 256 threads = 16 token rows x 16 vectors of 8
// channels; kTrips = row_block / 16 rows per thread.  The block is read twice, the second time from L2.
template <int kTrips>
__global__ void __launch_bounds__(256) quant_block_kernel(const QuantParams p) {
    __shared__ float warp_max[8];
    const int blk = blockIdx.x, head = blockIdx.y, batch = blockIdx.z;
    const int c = threadIdx.x & 15, r0 = threadIdx.x >> 4;
    const int first = blk * p.row_block;
    const int count = min(p.row_block, p.seq - first);
    const uint16_t* base = static_cast<const uint16_t*>(p.x) + batch * p.stride[0] + head * p.stride[1];
    float amax = 0.0f;
#pragma unroll
    for (int tr = 0; tr < kTrips; ++tr) {
        const int r = tr * 16 + r0;
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (r < count) raw = *reinterpret_cast<const uint4*>(base + (first + r) * p.stride[2] + c * 8);
        float f[8];
        unpack8(raw, p.is_bf16, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = warp_max[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) amax = fmaxf(amax, warp_max[i]);
    const float scale = amax > 0.0f ? amax / kE4m3Max : 1.0f;
    const float inv = 1.0f / scale;
    if (threadIdx.x == 0)
        p.scales[(static_cast<int64_t>(batch) * p.heads + head) * p.blocks + blk] = scale;
    uint8_t* obase = p.out + ((static_cast<int64_t>(batch) * p.heads + head) * p.seq) * 128;
#pragma unroll
    for (int tr = 0; tr < kTrips; ++tr) {
        const int r = tr * 16 + r0;
        if (r < count) {
            const uint4 raw = *reinterpret_cast<const uint4*>(base + (first + r) * p.stride[2] + c * 8);
            float f[8];
            unpack8(raw, p.is_bf16, f);
            *reinterpret_cast<uint2*>(obase + static_cast<int64_t>(first + r) * 128 + c * 8) = quant8(f, inv);
        }
    }
}

// mode 1, pass 1: per-channel absmax.  Grid (token chunk, head, batch).  Non-negative floats
// order like their bit patterns, so the running maximum is an integer atomicMax.
__global__ void __launch_bounds__(256) quant_channel_absmax_kernel(const QuantParams p, int rows_per_cta) {
    __shared__ float red[16][128];
    const int head = blockIdx.y, batch = blockIdx.z;
    const int c = threadIdx.x & 15, r0 = threadIdx.x >> 4;
    const int first = blockIdx.x * rows_per_cta;
    const int count = min(rows_per_cta, p.seq - first);
    const uint16_t* base = static_cast<const uint16_t*>(p.x) + batch * p.stride[0] + head * p.stride[1];
    float amax[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = r0; r < count; r += 16) {
        const uint4 raw = *reinterpret_cast<const uint4*>(base + (first + r) * p.stride[2] + c * 8);
        float f[8];
        unpack8(raw, p.is_bf16, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) amax[i] = fmaxf(amax[i], fabsf(f[i]));
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) red[r0][c * 8 + i] = amax[i];
    __syncthreads();
    if (threadIdx.x < 128) {
        float m = 0.0f;
#pragma unroll
        for (int g = 0; g < 16; ++g) m = fmaxf(m, red[g][threadIdx.x]);
        atomicMax(reinterpret_cast<unsigned int*>(p.scales) + (static_cast<int64_t>(batch) * p.heads + head) * 128 + threadIdx.x,
                  __float_as_uint(m));
    }
}

__global__ void quant_channel_finish_kernel(float* scales, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const float a = scales[i];
        scales[i] = a > 0.0f ? a / kE4m3Max : 1.0f;
    }
}

// mode 1, pass 2.
__global__ void __launch_bounds__(256) quant_channel_apply_kernel(const QuantParams p, int rows_per_cta) {
    const int head = blockIdx.y, batch = blockIdx.z;
    const int c = threadIdx.x & 15, r0 = threadIdx.x >> 4;
    const int first = blockIdx.x * rows_per_cta;
    const int count = min(rows_per_cta, p.seq - first);
    const uint16_t* base = static_cast<const uint16_t*>(p.x) + batch * p.stride[0] + head * p.stride[1];
    const float* sc = p.scales + (static_cast<int64_t>(batch) * p.heads + head) * 128 + c * 8;
    float inv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) inv[i] = 1.0f / sc[i];
    uint8_t* obase = p.out + ((static_cast<int64_t>(batch) * p.heads + head) * p.seq) * 128;
    for (int r = r0; r < count; r += 16) {
        const uint4 raw = *reinterpret_cast<const uint4*>(base + (first + r) * p.stride[2] + c * 8);
        float f[8];
        unpack8(raw, p.is_bf16, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] *= inv[i];
        *reinterpret_cast<uint2*>(obase + static_cast<int64_t>(first + r) * 128 + c * 8) = quant8(f, 1.0f);
    }
}

}  // namespace
}  // namespace sdb

using namespace sdb;

extern "C" int mindiesd_fa_block_quant(const mindiesd_quant_args* a, void* stream_) {
    if (!a || !a->x || !a->out || !a->scales) return MINDIESD_E_NULL;
    if (a->head_dim != 128) return MINDIESD_E_SHAPE;
    if (a->batch <= 0 || a->heads <= 0 || a->seq <= 0) return MINDIESD_E_SHAPE;
    if (a->batch > 65535 || a->heads > 65535) return MINDIESD_E_SHAPE;
    if (a->dtype != MINDIESD_BF16 && a->dtype != MINDIESD_FP16) return MINDIESD_E_DTYPE;
    if (reinterpret_cast<uintptr_t>(a->x) % 16 || reinterpret_cast<uintptr_t>(a->out) % 8) return MINDIESD_E_STRIDE;
    for (int i = 0; i < 3; ++i)
        if (a->x_stride[i] < 0 || a->x_stride[i] % 8) return MINDIESD_E_STRIDE;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    QuantParams p;
    p.x = a->x;
    p.out = static_cast<uint8_t*>(a->out);
    p.scales = a->scales;
    for (int i = 0; i < 3; ++i) p.stride[i] = a->x_stride[i];
    p.heads = a->heads;
    p.seq = a->seq;
    p.is_bf16 = a->dtype == MINDIESD_BF16;
    if (a->mode == 1 && a->rotate) return MINDIESD_E_VALUE;  // v is never rotated
    if (a->mode == 0) {
        if (a->row_block != 128 && a->row_block != 256 && a->row_block != 512) return MINDIESD_E_SHAPE;
        p.row_block = a->row_block;
        p.blocks = (a->seq + a->row_block - 1) / a->row_block;
        dim3 grid(p.blocks, a->heads, a->batch);
        // The rotation is a 128x128 product: it runs on the tensor cores inside the quantiser.
        if (a->rotate)
            return hadamard_quant_launch(a->x, a->x_stride, a->dtype, a->batch, a->heads, a->seq, a->row_block, a->out,
                                         a->scales, stream);
        if (a->row_block == 128) quant_block_kernel<8><<<grid, 256, 0, stream>>>(p);
        else if (a->row_block == 256) quant_block_kernel<16><<<grid, 256, 0, stream>>>(p);
        else quant_block_kernel<32><<<grid, 256, 0, stream>>>(p);
    } else if (a->mode == 1) {
        p.row_block = 0;
        p.blocks = 0;
        const int n = a->batch * a->heads * 128;
        cudaError_t e = cudaMemsetAsync(a->scales, 0, sizeof(float) * n, stream);
        if (e != cudaSuccess) return static_cast<int>(e);
        const int rows_per_cta = 256;
        dim3 grid((a->seq + rows_per_cta - 1) / rows_per_cta, a->heads, a->batch);
        quant_channel_absmax_kernel<<<grid, 256, 0, stream>>>(p, rows_per_cta);
        quant_channel_finish_kernel<<<(n + 255) / 256, 256, 0, stream>>>(a->scales, n);
        quant_channel_apply_kernel<<<grid, 256, 0, stream>>>(p, rows_per_cta);
    } else {
        return MINDIESD_E_VALUE;
    }
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? MINDIESD_OK : static_cast<int>(e);
}

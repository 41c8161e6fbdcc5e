// Kernel-side parameter block of the attention forward kernel and its launcher.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace sdb {

constexpr int kMaxKvBlocks = 4096;  // key/value blocks of 128 tokens one launch can walk (512 Ki tokens)

// Status codes written to the device status word by kernels whose bounded waits gave up.
constexpr int kStatusFaWaitGaveUp = 101;

struct FaParams {
    // Rank-4 tiled tensor maps over (channel, token, head, batch); box = 128 bytes x 128 tokens.
    alignas(64) CUtensorMap tm_q;
    alignas(64) CUtensorMap tm_k;
    alignas(64) CUtensorMap tm_v;
    void* out;
    float* lse;
    int64_t o_stride[3];  // element strides of batch, head, token
    int batch, heads, kv_heads, seq_q, seq_kv;
    int q_blocks, kv_blocks;
    int in_dtype;   // 0 bf16, 1 fp16, 3 e4m3
    int out_dtype;  // 0 bf16, 1 fp16, 2 fp32
    float scale_log2;  // softmax scale * log2(e)

    int sparse_mode;  // 0 dense, 1 int8 mask, 2 compacted list
    const int8_t* block_mask;
    int64_t mask_stride[3];
    const int64_t* select_idx;
    const int64_t* select_num;
    int64_t select_stride;  // elements between consecutive (q-block, head) rows of select_idx

    const float* q_scale;
    const float* k_scale;
    const float* v_scale;
    int k_scale_block, k_scale_count;
    int v_scale_block, v_scale_count;

    int* status;
};

int fa_fwd_smem_bytes(bool fp8);
cudaError_t fa_fwd_launch(const FaParams& p, cudaStream_t stream);

}  // namespace sdb

// Kernel-side parameter block of the attention forward kernel and its launcher.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace sdb {

constexpr int kMaxKvBlocks = 4096;  // key/value blocks of 128 tokens one launch can walk (512 Ki tokens)

// Status codes written to the device status word by kernels whose bounded waits gave up.
constexpr int kStatusFaWaitGaveUp = 101;

// Default time limit, in microseconds, of the bounded waits inside the kernels.
constexpr uint32_t kDefaultWaitLimitUs = 1000000u;

struct FaParams {
    // Rank-4 tiled tensor maps over (channel, token, head, batch); box = 128 bytes x 128 tokens.
    alignas(64) CUtensorMap tm_q;
    alignas(64) CUtensorMap tm_k;
    alignas(64) CUtensorMap tm_v;
    // RainFusion window permutation inside the kernel.  perm_on 1: q, k, v and out are in their original
    // token order, the kernel walks the permuted order (maps with a box of 128 bytes x 8 tokens below).
    // perm_on 2: q, k, v are already permuted; only the output rows go back to their original positions.
    alignas(64) CUtensorMap tm_q8;
    alignas(64) CUtensorMap tm_k8;
    alignas(64) CUtensorMap tm_v8;
    int perm_on, perm_t, perm_h, perm_w, perm_txt;
    void* out;
    float* lse;
    int64_t lse_stride[3];  // element strides of batch, head, token
    int64_t o_stride[3];  // element strides of batch, head, token
    int batch, heads, kv_heads, seq_q, seq_kv;
    int q_blocks, kv_blocks;
    int in_dtype;   // 0 bf16, 1 fp16, 3 e4m3
    int out_dtype;  // 0 bf16, 1 fp16, 2 fp32
    float scale_log2;  // softmax scale * log2(e)

    int causal;  // query i sees key j iff j <= i + (seq_kv - seq_q), per sequence
    // Packed variable-length sequences (batch 1): cumulative token counts [num_seqs + 1] on the device;
    // seq_q / seq_kv are then the totals.  NULL: one sequence per batch entry.
    const int32_t* cu_seqlens_q;
    const int32_t* cu_seqlens_kv;
    int num_seqs;

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
    uint32_t wait_limit_us;  // time limit of every bounded wait of this launch
    int test_withhold;       // failure injection for tests: the loader withholds its first copy
    // [B, N, grid.x, 2] 128-row query blocks of each thread block's two tiles (second -1: none), or null:
    // neighbouring blocks.  With it the launch has q_pair_count thread blocks per head.
    const int32_t* q_pairs;
    int q_pair_count;
};

int fa_fwd_smem_bytes(bool fp8);
cudaError_t fa_fwd_launch(const FaParams& p, cudaStream_t stream);

}  // namespace sdb

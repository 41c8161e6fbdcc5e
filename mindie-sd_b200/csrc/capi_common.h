// Helpers shared by the extern "C" entry points: tensor-map encoding and the per-device status word.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "../../include/mindiesd_b200.h"

namespace sdb {

constexpr int kMaxMaskBlocks = 2048;  // 128-token blocks per sequence the mask builder accepts (256 Ki tokens)

// Device address of the status word of the current device (NULL if the runtime refuses).
int* device_status_word();

inline int dtype_bytes(int dtype) {
    switch (dtype) {
        case MINDIESD_BF16:
        case MINDIESD_FP16: return 2;
        case MINDIESD_FP32: return 4;
        case MINDIESD_E4M3: return 1;
        default: return 0;
    }
}

// Encodes a rank-4 tiled tensor map over (channel, token, head, batch) of a tensor addressed by
// element strides {batch, head, token} with unit channel stride.  The box is 128 bytes of
// channels by box_rows tokens; 128-byte swizzle; out-of-range elements read as zero.
// Returns MINDIESD_OK or a MINDIESD_E_* code.
int encode_tile_map(CUtensorMap* map, const void* base, int dtype, int64_t channels, int64_t tokens,
                    int64_t heads, int64_t batch, const int64_t stride[3], int box_rows);

// e4m3 block quantisation of x @ rot (rot: [128, 128] in x's type), the product kept in tensor memory.
// The stored scale is absmax / 448 * post_scale.
int rotate_quant_launch(const void* x, const int64_t x_stride[3], const void* rot, int dtype, int batch, int heads, int seq,
                        int row_block, void* out, float* scales, float post_scale, cudaStream_t stream);
// The same with the fixed 128-point Hadamard rotation (an exact +-1 matrix, 1/sqrt(128) in the scale).
int hadamard_quant_launch(const void* x, const int64_t x_stride[3], int dtype, int batch, int heads, int seq, int row_block,
                          void* out, float* scales, cudaStream_t stream);

// Pooling + mask kernels of the RainFusion mask builder with the pooled means in `pooled`.
int rf_block_mask_impl(const mindiesd_mask_args* a, float* pooled, size_t pooled_bytes, cudaStream_t stream);

}  // namespace sdb

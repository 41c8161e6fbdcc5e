/*
 * C ABI of the B200 (sm_100a) attention hot path behind the MindIE-SD layer API.
 *
 * Every entry point takes plain device pointers and sizes, enqueues its kernels on the CUDA
 * stream it is given (a cudaStream_t passed as void*; NULL = the default stream) and returns
 * without synchronising.  Return value: 0 = enqueued; negative = invalid argument
 * (MINDIESD_E_*); positive = a cudaError_t raised by the launch.  No exception crosses this
 * boundary and inputs are never written.  Unless stated otherwise an entry point allocates
 * nothing; scratch memory is supplied by the caller.
 *
 * The reference interface each entry point stands in for is cited by its path inside the
 * MindIE-SD source tree.
 */
#ifndef MINDIESD_B200_H_
#define MINDIESD_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MINDIESD_B200_ABI_VERSION 3

enum {
    MINDIESD_OK = 0,
    MINDIESD_E_NULL = -1,     /* a required pointer is NULL                                  */
    MINDIESD_E_SHAPE = -2,    /* unsupported size (head_dim, block size, block count ...)    */
    MINDIESD_E_DTYPE = -3,    /* unsupported element type combination                        */
    MINDIESD_E_STRIDE = -4,   /* stride/pointer not aligned as the TMA engine requires       */
    MINDIESD_E_VALUE = -5,    /* scalar argument out of range                                */
    MINDIESD_E_DRIVER = -6,   /* the CUDA driver refused a tensor-map or attribute request   */
    MINDIESD_E_CAPACITY = -7  /* size exceeds a fixed capacity of the entry point            */
};

enum { MINDIESD_BF16 = 0, MINDIESD_FP16 = 1, MINDIESD_FP32 = 2, MINDIESD_E4M3 = 3 };

/* Block-sparsity source for mindiesd_attention_fwd. */
enum {
    MINDIESD_SPARSE_NONE = 0, /* dense                                                         */
    MINDIESD_SPARSE_MASK = 1, /* int8 mask [B, N, q_blocks, kv_blocks], non-zero = attend      */
    MINDIESD_SPARSE_LIST = 2  /* ascending int64 block ids [q_blocks, N, kv_blocks] + counts   */
};

/*
 * Attention forward:  out = softmax(scale * q k^T  [restricted to kept 128x128 blocks]) v.
 *
 * Tensors are addressed as [batch, head, token, channel] through element strides, so BNSD,
 * BSND and TND (batch = 1) are all expressed without copies; the channel stride is 1.
 * q/k/v: bf16 or fp16 (in_dtype), or e4m3 with dequantisation scales (see below).
 * out:   in_dtype, or fp32 (out_dtype = MINDIESD_FP32); for e4m3 inputs bf16/fp16/fp32.
 * lse:   optional fp32 [B, N, seq_q] natural-log-sum-exp of the scaled scores (NULL = skip).
 * Rows whose every block is masked produce zeros (lse = -inf).
 *
 * Stands in for: torch_npu.npu_prompt_flash_attention / npu_fusion_attention as called by
 * mindiesd/layers/flash_attn/prompt_flash_attn.py:48-57 and fused_attn_score.py:48-57;
 * aclnnLaserAttention launched by csrc/plugin/la.cpp:54-56; aclnnBlockSparseAttention launched
 * by csrc/plugin/block_sparse_attention.cpp:97-118 (MINDIESD_SPARSE_MASK);
 * aclnnRainFusionAttention launched by csrc/plugin/rainfusionattention.cpp:60-62
 * (MINDIESD_SPARSE_LIST); npu_fused_infer_attention_score_v2 with quant mode 7 as called by
 * mindiesd/quantization/layer.py:304-316 (in_dtype = MINDIESD_E4M3).
 */
typedef struct mindiesd_attn_args {
    const void* q;
    const void* k;
    const void* v;
    void* out;
    float* lse;
    int32_t batch, heads, kv_heads, seq_q, seq_kv, head_dim;
    int64_t q_stride[3]; /* element strides of batch, head, token */
    int64_t k_stride[3];
    int64_t v_stride[3];
    int64_t o_stride[3];
    int32_t in_dtype;
    int32_t out_dtype;
    float scale;

    int32_t sparse_mode;
    int32_t block_size;         /* must be 128 when sparse_mode != NONE */
    const int8_t* block_mask;   /* MASK: element strides of batch, head, q-block; kv-block stride 1 */
    int64_t mask_stride[3];
    const int64_t* select_idx;  /* LIST: [q_blocks, heads, kv_blocks], -1 padded, batch-invariant */
    const int64_t* select_num;  /* LIST: [q_blocks, heads] */

    /* e4m3 inputs only: real value = stored value * scale.
       q_scale [B, N, ceil(seq_q / 128)], k_scale [B, Nkv, ceil(seq_kv / k_scale_block)],
       v_scale [B, Nkv, head_dim] when v_scale_block == 0 (one scale per channel), else
       [B, Nkv, ceil(seq_kv / v_scale_block)].  Scale blocks are 128, 256 or 512 tokens. */
    const float* q_scale;
    const float* k_scale;
    const float* v_scale;
    int32_t k_scale_block;
    int32_t v_scale_block;

    /* Element strides of batch, head and token of lse; all zero = contiguous [B, N, seq_q]. */
    int64_t lse_stride[3];

    /* causal != 0: query i attends to key j only if j <= i + (seq_kv - seq_q), i.e. the triangle is
       aligned to the last query and the last key (for seq_q == seq_kv the usual lower triangle).
       This is sparse_mode 3 of npu_fusion_attention as mindiesd/layers/flash_attn/
       attention_forward_varlen.py:133-149 calls it, and the in-block triangle of
       ada_block_sparse_attention_cpu, tests/plugin/test_adablocksparseattention.py:69-72.  It combines
       with a block mask or list (a block is walked if both allow it).  Rows that see no key give zeros. */
    int32_t causal;

    /* num_seqs > 0: q is [1, N, Tq, D] and k, v are [1, Nkv, Tk, D] holding num_seqs sequences packed
       along the token axis (the TND layout of attention_forward_varlen, batch must be 1, seq_q = Tq,
       seq_kv = Tk); cu_seqlens_q / cu_seqlens_kv are int32 device arrays [num_seqs + 1] of cumulative
       token counts starting at 0.  Sequence i attends only to its own keys; with causal the triangle is
       aligned per sequence.  One launch covers all sequences and the host never reads the arrays.
       Not combined with a block mask / list or with e4m3 operands (MINDIESD_E_VALUE). */
    int32_t num_seqs;
    const int32_t* cu_seqlens_q;
    const int32_t* cu_seqlens_kv;

    /* perm_t > 0: q, k, v and out are in the ORIGINAL token order of a (perm_t, perm_h, perm_w) latent grid
       with perm_txt leading text tokens (seq_q == seq_kv == perm_txt + t*h*w), and the kernel applies the
       RainFusion window permutation on the fly: its tiles -- and therefore the rows and columns of the block
       mask / lists -- are those of the permuted order, its loads fetch each eight-token run of that order
       from where it lies, and its output rows go back to their original positions.  This replaces the
       four materialised permutations around the block-sparse call (rearrange_with_remaining of q, k, v and
       inv_rearrange_with_remaining / _bsa_inv_rearrange of the output,
       mindiesd/layers/flash_attn/sparse_flash_attn_rf_v2.py:137-289, sparse_flash_attn_rf_v3.py:22-97).
       Needs w and perm_txt to be multiples of 8 (MINDIESD_E_SHAPE otherwise: use mindiesd_rf_rearrange),
       two-byte operands, no packed sequences.
       perm_inputs_permuted != 0: q, k and v are ALREADY in the permuted order (mindiesd_rf_rearrange) and only
       the output is written back in the original order -- the inverse permutation costs nothing then, and
       any grid is accepted.  Fetching the permuted order on the fly costs 32 small copies per 128-token tile
       instead of 2 large ones: measured at the 21x45x80 grid it is slower than permuting q, k and v once, so
       the layer API permutes the inputs and lets the kernel undo the permutation of the output. */
    int32_t perm_t, perm_h, perm_w, perm_txt;
    int32_t perm_inputs_permuted;

    /* Time limit of every bounded wait inside the kernel, microseconds; 0 = the default (1 s).  A wait
       that runs out makes its thread block unwind, fill its output rows with NaN and set the device
       status word (mindiesd_device_status). */
    uint32_t wait_limit_us;
    /* Test hook, 0 in production: non-zero makes the loader of every thread block withhold its first
       key block (the copy is neither started nor announced), so that the consumer's wait runs into
       wait_limit_us.  It exists to exercise the give-up path without faulting or hanging the GPU. */
    int32_t test_withhold;

    /* Block-sparse attention only (sparse_mode 1 or 2), optional.  A thread block of the kernel works on two
       128-row query blocks at once and walks the UNION of their key-block lists; the more the two lists
       differ, the more steps serve one of the two only.  q_pairs names, per (batch, head), which two query
       blocks share a thread block: int32 [batch, heads, q_pair_count, 2], every query block exactly once, -1
       as the second entry of a thread block that has one only (mindiesd_rf_pair_blocks builds the table from
       a block mask, pairing blocks whose lists overlap most).  Null: neighbouring blocks (2i, 2i+1), which is
       what the reference's kernels do too.  The result is the same either way, bit for bit: a query row walks
       its own key blocks in the same order whoever shares its thread block.  Measured at the 591-block
       RainFusion mask of a 21x45x80 grid (density 0.32): 17-19 % of the steps serve one tile with neighbouring
       blocks, 8-10 % with the table, and the launch gets 0.2-1.8 % shorter (two runs); building the table takes
       0.6 ms, so it pays, if at all, where mask and table are kept across steps.  Not combined with causal,
       packed sequences, e4m3 operands or perm_t without perm_inputs_permuted (MINDIESD_E_VALUE). */
    const int32_t* q_pairs;
    int32_t q_pair_count;
} mindiesd_attn_args;

int mindiesd_attention_fwd(const mindiesd_attn_args* args, void* stream);

/*
 * Pairs the 128-row query blocks of every (batch, head) of a block mask by the similarity of their key-block
 * lists, for mindiesd_attn_args.q_pairs: greedy, heaviest row first, each taking the free row with the largest
 * Jaccard overlap.  mask: int8 [batch, heads, q_blocks, kv_blocks] by element strides (non-zero = kept);
 * pairs: int32 [batch, heads, (q_blocks + 1) / 2, 2] contiguous.  q_blocks, kv_blocks <= 1024.
 * No counterpart in the reference (its kernels take neighbouring blocks in index order,
 * csrc/ops/block_sparse_attention, csrc/ops/ada_block_sparse_attention).
 */
typedef struct mindiesd_pair_args {
    const int8_t* mask;
    int64_t mask_stride[3];
    int32_t batch, heads, q_blocks, kv_blocks;
    int32_t* pairs;
} mindiesd_pair_args;

int mindiesd_rf_pair_blocks(const mindiesd_pair_args* args, void* stream);

/*
 * RainFusion token permutation of the image tokens of a (t, h, w) latent grid into 8x8 spatial
 * windows (forward) and back (inverse = 1), text tokens moved from the front to the back
 * (forward) or back to the front (inverse).  src/dst: [B, N, S, D] by element strides, elements
 * of elem_bytes (1, 2 or 4) bytes, rows and strides multiples of 16 bytes, S = txt_len + t*h*w.
 * dst must not alias src.
 *
 * Stands in for rearrange_with_remaining / inv_rearrange_with_remaining /
 * do_tensor_inv_rearrange (mindiesd/layers/flash_attn/sparse_flash_attn_rf_v2.py:137-196,
 * 199-289, 321-337), _bsa_inv_rearrange and do_tensor_rearrange_only
 * (sparse_flash_attn_rf_v3.py:22-118).
 */
typedef struct mindiesd_rearrange_args {
    const void* src;
    void* dst;
    int32_t batch, heads, seq, head_dim, elem_bytes;
    int64_t src_stride[3];
    int64_t dst_stride[3];
    int32_t t, h, w, txt_len;
    int32_t inverse;
} mindiesd_rearrange_args;

int mindiesd_rf_rearrange(const mindiesd_rearrange_args* args, void* stream);

/*
 * RainFusion block-mask builder.  q and k are in their ORIGINAL token order; the window
 * permutation is applied in the index arithmetic.  Per head: mean of every 128-token block of
 * the permuted q and k (the tail block over its real length), block scores q_mean . k_mean,
 * keep the ceil(kv_blocks * (1 - sparsity)) largest of each row (every score equal to the
 * smallest kept one is kept too), then force the text blocks (last ceil(txt_len/128) rows and
 * columns) and, if protect_first_frame, the first ceil(h*w/128) rows and columns; if
 * temporal_band >= 0 also every block pair whose frame ranges lie within that many frames.
 * Outputs (each optional): mask int8 [B, N, qb, kb]; select_idx int64 [qb, N, kb] ascending,
 * -1 padded, and select_num int64 [qb, N], both taken from batch 0 as the reference does.
 * scratch: caller-supplied, at least mindiesd_rf_block_mask_scratch_bytes() bytes, 256-byte
 * aligned; holds the pooled means between the two kernels.
 *
 * Stands in for avgpool + get_blockwise_mask + get_mask_index
 * (mindiesd/layers/flash_attn/sparse_flash_attn_rf_v2.py:24-134).
 */
typedef struct mindiesd_mask_args {
    const void* q;
    const void* k;
    int32_t batch, heads, seq, head_dim;
    int64_t q_stride[3];
    int64_t k_stride[3];
    int32_t dtype; /* MINDIESD_BF16 / FP16 / FP32 */
    int32_t t, h, w, txt_len;
    int32_t block_size; /* 128 */
    float scale;        /* > 0; the kept set does not depend on its value */
    double sparsity;    /* in [0, 1); double so that ceil(kv_blocks * (1 - sparsity)) equals the reference's */
    int32_t protect_first_frame;
    int32_t temporal_band; /* < 0: off (the reference has no band) */
    int8_t* mask;
    int64_t* select_idx;
    int64_t* select_num;
    void* scratch;
    size_t scratch_bytes;
} mindiesd_mask_args;

size_t mindiesd_rf_block_mask_scratch_bytes(int32_t batch, int32_t heads, int32_t seq, int32_t head_dim);
int mindiesd_rf_block_mask(const mindiesd_mask_args* args, void* stream);

/*
 * The same mask builder for hosts that cannot allocate device memory.  It has no counterpart in
 * the reference, whose operators take a fresh workspace tensor from the framework on every call.
 * Some hosts of this library cannot do the equivalent: a C or C++ service that handed the whole
 * device to its own arena at start-up and forbids cudaMalloc afterwards, or a step loop in which a
 * cudaMalloc would stall the device.  For them the pooled means live in a 4 MiB array inside the
 * library's device image (every GPU that loads the library holds those 4 MiB until the process
 * exits); `scratch` and `scratch_bytes` of the arguments are ignored and the call allocates nothing.
 *
 * Limit: batch * heads * blocks * head_dim * 2 * sizeof(float) must fit in
 * mindiesd_rf_block_mask_static_capacity() bytes (blocks = ceil(t*h*w/128) + ceil(txt_len/128));
 * a larger problem returns MINDIESD_E_CAPACITY and must use mindiesd_rf_block_mask.
 * The first call on each device looks up the array's device address (the only set-up); make that
 * call before starting any stream capture.  All calls on a device share the one array: calls whose
 * kernels may overlap on the GPU (different streams without ordering) race and give wrong masks;
 * calls on one stream, or otherwise ordered, are safe.  Nothing needs clearing between calls.
 */
size_t mindiesd_rf_block_mask_static_capacity(void);
int mindiesd_rf_block_mask_static(const mindiesd_mask_args* args, void* stream);

/*
 * The two stages of the mask builder on their own, for callers that use the reference's helper
 * functions one at a time.
 *
 * mindiesd_rf_pool: fp32 means of 128-token blocks of x [B, N, S, D] -> pooled [B, N, blocks, D].
 * permute = 0 pools consecutive tokens (blocks = ceil(S/128)); permute = 1 pools the
 * window-permuted order of a (t, h, w) grid with txt_len leading text tokens, image and text
 * separately (blocks = ceil(t*h*w/128) + ceil(txt_len/128)).
 * Stands in for avgpool and the pooling half of do_tensor_rearrange_pooling
 * (mindiesd/layers/flash_attn/sparse_flash_attn_rf_v2.py:24-73, 292-317).
 *
 * mindiesd_rf_mask_from_pooled: the mask / block lists from pooled q and k (fp32, contiguous
 * [B, N, blocks, D]).  Stands in for get_blockwise_mask + get_mask_index (rf_v2.py:76-134).
 */
typedef struct mindiesd_pool_args {
    const void* x;
    float* pooled;
    int32_t batch, heads, seq, head_dim;
    int64_t x_stride[3];
    int32_t dtype;
    int32_t t, h, w, txt_len;
    int32_t permute;
    int32_t block_size; /* 128 */
} mindiesd_pool_args;

int mindiesd_rf_pool(const mindiesd_pool_args* args, void* stream);

typedef struct mindiesd_pooled_mask_args {
    const float* q_pooled;
    const float* k_pooled;
    int32_t batch, heads, blocks, head_dim;
    int32_t t, h, w, txt_len;
    int32_t block_size; /* 128 */
    int32_t protect_first_frame;
    int32_t temporal_band;
    double sparsity;
    int8_t* mask;
    int64_t* select_idx;
    int64_t* select_num;
} mindiesd_pooled_mask_args;

int mindiesd_rf_mask_from_pooled(const mindiesd_pooled_mask_args* args, void* stream);

/*
 * Dynamic block quantisation to e4m3 for attention operands.  x: [B, N, S, D] bf16/fp16 by
 * element strides.  mode 0: one scale per (row_block tokens x 128 channels) block,
 * scale = absmax / 448 (1 where the block is all zero), scales fp32 [B, N, ceil(S/row_block)];
 * mode 1: one scale per channel over the whole sequence, scales fp32 [B, N, D].
 * out: e4m3 [B, N, S, D] contiguous.
 * rotate: q and k rotated by the same orthogonal matrix give the same q k^T; the rotation spreads
 * outlier channels so that the e4m3 rounding error of the scores stays small.  It fuses the
 * reference's `query @ q_rot` / `key @ k_rot` (mindiesd/quantization/layer.py:284-285) into the
 * quantisation pass for the fixed Hadamard rotation.
 *
 * Stands in for torch_npu.npu_dynamic_block_quant as called by fa_block_quant_preprocess
 * (mindiesd/layers/quant/block_quant.py:43-46).
 */
typedef struct mindiesd_quant_args {
    const void* x;
    void* out;
    float* scales;
    int32_t batch, heads, seq, head_dim;
    int64_t x_stride[3];
    int32_t dtype;
    int32_t mode;
    int32_t row_block; /* 128, 256 or 512 (mode 0) */
    int32_t rotate;    /* mode 0: first rotate every token by the 128-point Walsh-Hadamard matrix / sqrt(128) */
} mindiesd_quant_args;

int mindiesd_fa_block_quant(const mindiesd_quant_args* args, void* stream);

/*
 * Rotation by a learned matrix fused with the block quantisation:  y = x rot  per token
 * (rot: [128, 128] row-major, the type of x), then mode-0 quantisation of y as above, the scale taken
 * on the fp32 products.  y is never written: 2 bytes in, 1 byte out per element.
 *
 * Stands in for `query @ self.q_rot` / `key @ self.k_rot` followed by fa_block_quant_preprocess
 * (mindiesd/quantization/layer.py:284-302).
 */
typedef struct mindiesd_rotate_quant_args {
    const void* x;   /* [B, N, S, 128] bf16/fp16 by element strides */
    const void* rot; /* [128, 128] contiguous */
    void* out;       /* e4m3 [B, N, S, 128] contiguous, 16-byte aligned */
    float* scales;   /* fp32 [B, N, ceil(S/row_block)] */
    int32_t batch, heads, seq, head_dim; /* head_dim 128 */
    int64_t x_stride[3];
    int32_t dtype;
    int32_t row_block; /* 128, 256 or 512 */
} mindiesd_rotate_quant_args;

int mindiesd_fa_rotate_quant(const mindiesd_rotate_quant_args* args, void* stream);

/*
 * Sparse block estimate: the mask builder of adaptive block-sparse attention ("ada_bsa").
 *
 * Tokens are taken `stride` (8) at a time; the pooled logit of query group g and key group h is
 * scale * sum_i q[8g + 7 - i] . k[8h + i].  Each row of pooled logits goes through a softmax over
 * all key groups; the probabilities are summed over the 16 x 16 groups of every 128 x 128 token
 * block.  Per query block, with the last key block's mass cleared (keep_recent), the heaviest key
 * blocks are kept until their running sum reaches `threshold` of the row's total -- at most
 * int(row_sparse * blocks) of them when row_sparse * blocks is smaller than that prefix -- together
 * with every block as heavy as the last one kept, the first block (keep_sink) and the last block
 * (keep_recent).
 *
 *   q, k:   bf16 or fp16, addressed [batch, head, token, channel] through element strides
 *   seq:    a multiple of 8 (the golden pads the last group with zero tokens; a caller with a
 *           ragged sequence does the same before the call)
 *   mask:   int8 [batch, heads, blocks, mask_cols], mask_cols >= blocks (the reference rounds it
 *           up to a multiple of 32); columns >= blocks are written 0
 *   count:  int32 [batch, heads, blocks]: kept blocks per row
 *   scratch: at least mindiesd_sparse_block_estimate_scratch_bytes(1, 1, seq) bytes (one head per
 *           pass); the size that function returns for the real batch and heads lets four heads
 *           run per pass, whose partial sums stay in L2
 * causal != 0 follows the golden's causal branch (:73-76, 129-143): the queries of a 1024-token chunk take
 * their softmax over the keys up to the end of that chunk, a query block ranks the key blocks up to its
 * own with its own block's mass cleared (it is kept only if the guard is 0), rows 0 and 1 keep every
 * block up to their own, the first block always stays, the cap is int(row_sparse * (row + 1)), and
 * blocks beyond the row's own are 0.  keep_recent has no effect then.
 *
 * Stands in for: aclnnSparseBlockEstimate as registered in csrc/plugin/register_ops.cpp:46-53 and
 * called by mindiesd/layers/flash_attn/sparse_flash_attn_ada_bsa.py:31-47; semantics pinned by
 * sparse_estimate_cpu, tests/plugin/test_sparseblockestimate.py:49-145.
 */
typedef struct mindiesd_estimate_args {
    const void* q;
    const void* k;
    int64_t q_stride[3]; /* elements: batch, head, token */
    int64_t k_stride[3];
    int32_t dtype; /* MINDIESD_BF16 / MINDIESD_FP16 */
    int32_t batch, heads, kv_heads, seq, head_dim; /* head_dim 64 or 128 */
    int32_t stride;      /* 8 */
    int32_t sparse_size; /* 128 */
    float scale;         /* multiplies the pooled dot product; the layer passes softmax_scale / stride */
    float threshold;     /* share of a row's mass the kept prefix must reach */
    double row_sparse;   /* cap on the kept prefix as a share of the row; <= 0 or >= 1: no cap */
    int32_t causal;
    int32_t keep_sink, keep_recent;
    int8_t* mask;
    int32_t mask_cols;
    int32_t* count;
    void* scratch;
    size_t scratch_bytes;
    /* causal only: key tokens that exist when `seq` was rounded up to a multiple of 8 with zero tokens --
       the golden drops a trailing partial group of keys in its causal branch (:73-76); 0 = seq. */
    int32_t causal_key_tokens;
} mindiesd_estimate_args;

size_t mindiesd_sparse_block_estimate_scratch_bytes(int32_t batch, int32_t heads, int32_t seq);
int mindiesd_sparse_block_estimate(const mindiesd_estimate_args* args, void* stream);

/*
 * Rotary position embedding:  out = x * cos + rotated(x) * sin  per token, with
 * mode 1 ("rotated_half"):        rotated(x) = (-x[d/2:], x[:d/2])
 * mode 2 ("rotated_interleaved"): rotated(x) = (-x1, x0, -x3, x2, ...).
 * x/out: [B, N, S, D] by element strides (unit channel stride), bf16, fp16 or fp32, D even.
 * cos/sin: contiguous [S, D] tables, fp32 or the type of x.  The arithmetic runs in the tables' type
 * (fp32: both products and the sum rounded to fp32, one rounding to the type of x at the end), which is
 * the reference's unfused formula bit for bit.  out may alias x when mode == 2 only.
 *
 * Stands in for torch_npu.npu_rotary_mul as called by rotary_position_embedding
 * (mindiesd/layers/rope.py:54-115).
 */
typedef struct mindiesd_rope_args {
    const void* x;
    void* out;
    const void* cos;
    const void* sin;
    int32_t batch, heads, seq, head_dim;
    int64_t x_stride[3];   /* element strides of batch, head, token */
    int64_t out_stride[3];
    int32_t dtype;         /* MINDIESD_BF16 / FP16 / FP32 */
    int32_t table_dtype;   /* MINDIESD_FP32 or dtype */
    int32_t mode;          /* 1 half, 2 interleaved */
} mindiesd_rope_args;

int mindiesd_rope(const mindiesd_rope_args* args, void* stream);

/*
 * The re-shard step of Ulysses sequence parallelism as one data-movement kernel.
 *
 * A rank holds `rows` tokens with all N heads: tensors [rows, N, 128] addressed by a row and a head
 * stride.  Rank r of `world` owns the heads [r * group_heads, (r + 1) * group_heads); a call moves
 * the piece [head0, head0 + heads) of every rank's group.
 *
 * inverse == 0 (before attention): for every destination rank r the piece of tensor[0..n_src-1] (q, k, v)
 *   is written to table[r] as [rows, n_src * heads, 128] (row stride table_row_stride, tensor i at head
 *   slot i * heads).  table[r] may be chunk r of a local send buffer, or an address inside rank r's
 *   receive buffer mapped into this process (peer memory): then the kernel IS the all-to-all, its
 *   stores crossing NVLink.  With rope_mode != 0, tensor[0] and tensor[1] are rotated on the way by the
 *   rotary embedding (fp32 tables [rows, 128] for this rank's tokens, arithmetic as mindiesd_rope).
 * inverse == 1 (after attention): table[r] holds rank r's [rows, heads, 128] output block for this
 *   rank's tokens; it is written to tensor[0][row, r * group_heads + head0 + j].
 *
 * bf16 / fp16, head_dim 128, every pointer and stride a multiple of 16 bytes.
 * thread_blocks: how many to launch (0 = enough to fill the GPU); a small number leaves the SMs to an
 * attention kernel running beside it.
 *
 * Stands in for the reshapes and the two torch.distributed all_to_all calls of the Ulysses pattern in
 * docs/zh/features/parallelism.md:207-233, and, with rope_mode, for rotary_position_embedding
 * (mindiesd/layers/rope.py:54-115) on q and k before them.
 */
#define MINDIESD_MAX_RANKS 8

typedef struct mindiesd_ulysses_move_args {
    const void* tensor[3];
    void* table[MINDIESD_MAX_RANKS];
    int64_t tensor_row_stride;  /* elements */
    int64_t tensor_head_stride;
    int64_t table_row_stride;
    int32_t n_src;              /* 1..3 (inverse: 1) */
    int32_t rows, world, group_heads, head0, heads, head_dim;
    int32_t dtype;
    int32_t inverse;
    const float* cos;
    const float* sin;
    int32_t rope_mode;          /* 0 none, 1 half, 2 interleaved */
    int32_t thread_blocks;
} mindiesd_ulysses_move_args;

int mindiesd_ulysses_move(const mindiesd_ulysses_move_args* args, void* stream);

/*
 * Peer memory for the sequence-parallel exchange (one process per GPU on one box).  mindiesd_peer_export
 * turns a device pointer of this process into a 64-byte handle plus the pointer's offset inside its
 * allocation; the other rank passes both to mindiesd_peer_open (with ITS device current) and gets an
 * address it may hand to mindiesd_ulysses_move as a table entry: stores to it and loads from it cross
 * NVLink.  An allocation is mapped once per process and stays mapped until the process exits; the
 * exporting rank must keep the allocation alive as long as any peer uses it.  Positive return values are
 * cudaError_t codes (e.g. no peer access between the two devices).
 * The reference has no counterpart: its documented Ulysses pattern moves everything through the
 * collective library (docs/zh/features/parallelism.md:207-233).
 */
int mindiesd_peer_export(const void* ptr, uint8_t handle[64], uint64_t* offset);
int mindiesd_peer_open(const uint8_t handle[64], uint64_t offset, void** ptr);

/*
 * Strided copy between pinned host memory and device memory (either direction, chosen by the
 * addresses) on a stream: `height` rows of `width_bytes`, rows `*_pitch` bytes apart.  It lets a
 * host-resident [rows, N, D] tensor be brought in one head range at a time, so that the first piece
 * of a sequence-parallel layer starts before the whole tensor has crossed PCIe.  The reference keeps
 * activations on the device and has no counterpart.
 */
int mindiesd_copy_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes,
                     size_t height, void* stream);

/*
 * Device status word of the current device: 0, or the code of the first bounded wait inside a
 * kernel that gave up since the last call.  Synchronises the device; clears the word.
 */
int mindiesd_device_status(void);

/*
 * The status word and its diagnostics without clearing them: out[0] code, out[1] number of the
 * wait that gave up first, out[2..4] index of the thread block that reported it.  Synchronises.
 */
int mindiesd_device_status_detail(int32_t out[8]);

int mindiesd_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* MINDIESD_B200_H_ */

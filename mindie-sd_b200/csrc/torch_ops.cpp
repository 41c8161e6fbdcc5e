// torch.ops.mindiesd.* for CUDA tensors.  The attention and estimator schemas are those of MindIE-SD's
// own operator library (csrc/plugin/register_ops.cpp:27-32, 41-67), argument names
// included, because callers pass every argument by keyword.  Each implementation checks its
// arguments, allocates its outputs from torch's caching allocator, and calls one extern "C"
// launcher of libmindiesd_b200.so on the current stream; nothing synchronises.
#include <cstdlib>
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <stdexcept>
#include <limits>
#include <string>
#include <tuple>
#include <vector>

#include "mindiesd_b200.h"

namespace {

int dtype_code(at::ScalarType t) {
    switch (t) {
        case at::kBFloat16: return MINDIESD_BF16;
        case at::kHalf: return MINDIESD_FP16;
        case at::kFloat: return MINDIESD_FP32;
        case at::kFloat8_e4m3fn: return MINDIESD_E4M3;
        default: TORCH_CHECK(false, "mindiesd: unsupported dtype ", t);
    }
}

const char* error_text(int rc) {
    switch (rc) {
        case MINDIESD_E_NULL: return "a required pointer is NULL";
        case MINDIESD_E_SHAPE: return "unsupported size";
        case MINDIESD_E_DTYPE: return "unsupported element type";
        case MINDIESD_E_STRIDE: return "stride or pointer not 16-byte aligned";
        case MINDIESD_E_VALUE: return "scalar argument out of range";
        case MINDIESD_E_DRIVER: return "the CUDA driver refused the request";
        case MINDIESD_E_CAPACITY: return "size exceeds a fixed capacity";
        default: return "CUDA error";
    }
}

void check_rc(int rc, const char* api) {
    TORCH_CHECK(rc == 0, "call ", api, " failed, detail: ", error_text(rc), " (code ", rc, ")");
}

void* stream_of(const at::Tensor& t) { return c10::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

// Element strides {batch, head, token} of a 4-D tensor whose dims are (B, N, S, D) when head_first,
// else (B, S, N, D).
void fill_strides(const at::Tensor& t, bool head_first, int64_t out[3]) {
    TORCH_CHECK(t.stride(3) == 1, "mindiesd: the channel dimension must be contiguous");
    out[0] = t.stride(0);
    out[1] = head_first ? t.stride(1) : t.stride(2);
    out[2] = head_first ? t.stride(2) : t.stride(1);
}

struct SparseSpec {
    int mode = MINDIESD_SPARSE_NONE;
    const at::Tensor* mask = nullptr;
    const at::Tensor* select_idx = nullptr;
    const at::Tensor* select_num = nullptr;
    const at::Tensor* q_pairs = nullptr;  // int32 [B, N, (q_blocks + 1) / 2, 2] from rf_pair_blocks, or none
};

// What only some operators pass on: the causal triangle, where the log-sum-exp goes, packed sequences.
struct AttnExtra {
    bool causal = false;
    int perm[4] = {0, 0, 0, 0};  // (t, h, w, txt_len): the window permutation applied inside the kernel
    bool perm_inputs_permuted = false;  // q, k, v already permuted: only the output goes back
    int64_t lse_stride[3] = {0, 0, 0};   // elements: batch, head, token; all zero = contiguous [B, N, S]
    const at::Tensor* cu_seqlens_q = nullptr;  // int32 [num_seqs + 1] on the device (q, k, v then have batch 1)
    const at::Tensor* cu_seqlens_kv = nullptr;
};

// q/k/v viewed as [B, *, *, D] in BNSD (head_first) or BSND order.  seq_q/seq_kv < 0: take from the view.
void run_attention(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, at::Tensor& out, float* lse,
                   bool head_first, double scale, const SparseSpec& sp, int64_t seq_q = -1, int64_t seq_kv = -1,
                   const at::Tensor* q_scale = nullptr, const at::Tensor* k_scale = nullptr,
                   const at::Tensor* v_scale = nullptr, int k_block = 0, int v_block = 0,
                   const AttnExtra& extra = AttnExtra()) {
    TORCH_CHECK(q.is_cuda() && k.is_cuda() && v.is_cuda(), "mindiesd: q, k, v must be CUDA tensors");
    TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4, "mindiesd: q, k, v must be 4-D");
    TORCH_CHECK(q.scalar_type() == k.scalar_type() && q.scalar_type() == v.scalar_type(),
                "mindiesd: q, k, v must share a dtype");
    const int sdim = head_first ? 2 : 1, ndim = head_first ? 1 : 2;
    mindiesd_attn_args a = {};
    a.q = q.data_ptr();
    a.k = k.data_ptr();
    a.v = v.data_ptr();
    a.out = out.data_ptr();
    a.lse = lse;
    a.batch = static_cast<int32_t>(q.size(0));
    a.heads = static_cast<int32_t>(q.size(ndim));
    a.kv_heads = static_cast<int32_t>(k.size(ndim));
    a.seq_q = static_cast<int32_t>(seq_q >= 0 ? seq_q : q.size(sdim));
    a.seq_kv = static_cast<int32_t>(seq_kv >= 0 ? seq_kv : k.size(sdim));
    a.head_dim = static_cast<int32_t>(q.size(3));
    TORCH_CHECK(k.size(0) == q.size(0) && v.size(0) == q.size(0) && k.size(3) == q.size(3) && v.size(3) == q.size(3) &&
                    v.size(sdim) == k.size(sdim) && v.size(ndim) == k.size(ndim),
                "mindiesd: q, k, v shapes are inconsistent");
    fill_strides(q, head_first, a.q_stride);
    fill_strides(k, head_first, a.k_stride);
    fill_strides(v, head_first, a.v_stride);
    fill_strides(out, head_first, a.o_stride);
    a.in_dtype = dtype_code(q.scalar_type());
    a.out_dtype = dtype_code(out.scalar_type());
    a.scale = static_cast<float>(scale);
    a.sparse_mode = sp.mode;
    a.block_size = 128;
    if (sp.mode == MINDIESD_SPARSE_MASK) {
        const at::Tensor& m = *sp.mask;
        TORCH_CHECK(m.is_cuda() && m.scalar_type() == at::kChar && m.dim() == 4 && m.stride(3) == 1,
                    "mindiesd: block_sparse_mask must be a CUDA int8 tensor [B, N, q_blocks, kv_blocks]");
        TORCH_CHECK(m.size(0) == a.batch && m.size(1) == a.heads && m.size(2) >= (a.seq_q + 127) / 128 &&
                        m.size(3) >= (a.seq_kv + 127) / 128,
                    "mindiesd: block_sparse_mask shape does not cover the sequence");
        a.block_mask = m.data_ptr<int8_t>();
        a.mask_stride[0] = m.stride(0);
        a.mask_stride[1] = m.stride(1);
        a.mask_stride[2] = m.stride(2);
    } else if (sp.mode == MINDIESD_SPARSE_LIST) {
        a.select_idx = sp.select_idx->data_ptr<int64_t>();
        a.select_num = sp.select_num->data_ptr<int64_t>();
    }
    if (q_scale) {
        a.q_scale = q_scale->data_ptr<float>();
        a.k_scale = k_scale->data_ptr<float>();
        a.v_scale = v_scale->data_ptr<float>();
        a.k_scale_block = k_block;
        a.v_scale_block = v_block;
    }
    a.causal = extra.causal ? 1 : 0;
    a.perm_t = extra.perm[0];
    a.perm_h = extra.perm[1];
    a.perm_w = extra.perm[2];
    a.perm_txt = extra.perm[3];
    a.perm_inputs_permuted = extra.perm_inputs_permuted ? 1 : 0;
    for (int i = 0; i < 3; ++i) a.lse_stride[i] = extra.lse_stride[i];
    if (extra.cu_seqlens_q) {
        const at::Tensor& cq = *extra.cu_seqlens_q;
        const at::Tensor& ck = *extra.cu_seqlens_kv;
        TORCH_CHECK(cq.is_cuda() && ck.is_cuda() && cq.scalar_type() == at::kInt && ck.scalar_type() == at::kInt &&
                        cq.dim() == 1 && ck.dim() == 1 && cq.is_contiguous() && ck.is_contiguous() &&
                        cq.numel() == ck.numel() && cq.numel() >= 2,
                    "mindiesd: cu_seqlens_q and cu_seqlens_k must be contiguous CUDA int32 vectors of one length >= 2");
        a.num_seqs = static_cast<int32_t>(cq.numel() - 1);
        a.cu_seqlens_q = cq.data_ptr<int32_t>();
        a.cu_seqlens_kv = ck.data_ptr<int32_t>();
    }
    c10::cuda::CUDAGuard guard(q.device());
    // Block mask, MINDIESD_PAIR_BLOCKS=1: the query blocks that share a thread block are chosen by the overlap
    // of their key-block lists (fewer steps that serve only one of the two); same result bit for bit.  Off by
    // default: at the 591-block RainFusion mask the attention gets 0.1-0.6 ms (0.2-1.8 %) shorter and building
    // the table costs 0.6 ms, so it can pay only where the caller keeps mask and table across steps (the C
    // ABI takes a ready table: mindiesd_attn_args.q_pairs).
    at::Tensor pairs;
    static const bool pair_blocks = [] {
        const char* e = std::getenv("MINDIESD_PAIR_BLOCKS");
        return e && e[0] == '1';
    }();
    const int q_blocks = (a.seq_q + 127) / 128, kv_blocks = (a.seq_kv + 127) / 128;
    if (sp.q_pairs) {
        const at::Tensor& t = *sp.q_pairs;
        TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kInt && t.is_contiguous() && t.dim() == 4 && t.size(0) == a.batch &&
                        t.size(1) == a.heads && t.size(2) == (q_blocks + 1) / 2 && t.size(3) == 2,
                    "mindiesd: q_pairs must be a contiguous CUDA int32 tensor [B, N, (q_blocks + 1) / 2, 2]");
        a.q_pairs = t.data_ptr<int32_t>();
        a.q_pair_count = (q_blocks + 1) / 2;
    } else if (pair_blocks && sp.mode == MINDIESD_SPARSE_MASK && !extra.causal && !extra.cu_seqlens_q && !q_scale &&
        (extra.perm[0] == 0 || extra.perm_inputs_permuted) && q_blocks >= 16 && q_blocks <= 1024 && kv_blocks <= 1024) {
        pairs = at::empty({a.batch, a.heads, (q_blocks + 1) / 2, 2}, q.options().dtype(at::kInt));
        mindiesd_pair_args pa = {};
        pa.mask = a.block_mask;
        for (int i = 0; i < 3; ++i) pa.mask_stride[i] = a.mask_stride[i];
        pa.batch = a.batch;
        pa.heads = a.heads;
        pa.q_blocks = q_blocks;
        pa.kv_blocks = kv_blocks;
        pa.pairs = pairs.data_ptr<int32_t>();
        check_rc(mindiesd_rf_pair_blocks(&pa, stream_of(q)), "mindiesd_rf_pair_blocks");
        a.q_pairs = pa.pairs;
        a.q_pair_count = (q_blocks + 1) / 2;
    }
    check_rc(mindiesd_attention_fwd(&a, stream_of(q)), "mindiesd_attention_fwd");
}

// Head dims below 128 (the reference's own shape list is mostly 40, 64, 88, 96: tests/plugin/test_la.csv) run
// on the 128-wide kernel with zero channels appended: zeros add nothing to q k^T and the extra output
// channels are cut off.  It costs a padded copy of q, k, v -- the reference's laser attention pads the
// same way (mindiesd/layers/flash_attn/ascend_laser_attention.py:38-75).
at::Tensor pad_head_dim(const at::Tensor& x) {
    const int64_t d = x.size(-1);
    if (d == 128) return x;
    TORCH_CHECK(d > 0 && d < 128, "mindiesd: head dim must be at most 128, got ", d);
    return at::constant_pad_nd(x, {0, 128 - d}, 0);
}

// ---- la: dense attention, fp32 output + log-sum-exp -----------------------------------------------
std::tuple<at::Tensor, at::Tensor> la_cuda(const at::Tensor& query, const at::Tensor& key, const at::Tensor& value,
                                           const c10::optional<at::Tensor>& atten_mask,
                                           const c10::optional<at::Tensor>& alibi_mask,
                                           const c10::optional<at::Tensor>& drop_mask, double scale_value,
                                           int64_t head_num, std::string input_layout, double keep_prob,
                                           int64_t pre_tokens, int64_t next_tokens, bool is_highPrecision) {
    if (query.dim() != 4) {
        throw std::invalid_argument("The first input dimension of la must be 4 but got " + std::to_string(query.dim()));
    }
    TORCH_CHECK(input_layout == "BNSD", "la: input_layout only supports 'BNSD'");
    TORCH_CHECK(!atten_mask.has_value() && !alibi_mask.has_value() && !drop_mask.has_value(),
                "la: atten_mask, alibi_mask and drop_mask are not supported");
    TORCH_CHECK(keep_prob == 1.0, "la: keep_prob must be 1.0");
    (void)head_num; (void)pre_tokens; (void)next_tokens; (void)is_highPrecision;
    at::Tensor lse = at::empty({query.size(0), query.size(1), query.size(2)}, query.options().dtype(at::kFloat));
    const int64_t d = query.size(3);
    at::Tensor q = pad_head_dim(query), k = pad_head_dim(key), v = pad_head_dim(value);
    at::Tensor out = at::empty(q.sizes(), q.options().dtype(at::kFloat));
    run_attention(q, k, v, out, lse.data_ptr<float>(), true, scale_value, SparseSpec{});
    if (d != 128) out = out.narrow(3, 0, d).contiguous();
    return std::make_tuple(lse, out);
}

// ---- block_sparse_attention: int8 block mask ---------------------------------------------------------
std::tuple<at::Tensor, at::Tensor> block_sparse_attention_cuda(
    const at::Tensor& query, const at::Tensor& key, const at::Tensor& value,
    const c10::optional<at::Tensor>& block_sparse_mask, at::IntArrayRef block_shape, std::string q_input_layout,
    std::string kv_input_layout, int64_t num_key_value_heads, double scale_value, int64_t inner_precise,
    c10::OptionalIntArrayRef actual_seq_lengths, c10::OptionalIntArrayRef actual_seq_lengths_kv,
    int64_t softmax_lse_flag) {
    TORCH_CHECK(q_input_layout == "TND" || q_input_layout == "BNSD",
                "block_sparse_attention: q_input_layout only supports 'TND' and 'BNSD', got ", q_input_layout);
    TORCH_CHECK(kv_input_layout == "TND" || kv_input_layout == "BNSD",
                "block_sparse_attention: kv_input_layout only supports 'TND' and 'BNSD', got ", kv_input_layout);
    TORCH_CHECK(q_input_layout == kv_input_layout,
                "block_sparse_attention: q_input_layout and kv_input_layout must be consistent.");
    TORCH_CHECK(q_input_layout != "TND" || (actual_seq_lengths.has_value() && actual_seq_lengths_kv.has_value()),
                "block_sparse_attention: actual_seq_lengths and actual_seq_lengths_kv are required for TND layout.");
    TORCH_CHECK(block_shape.size() == 2 && block_shape[0] == 128 && block_shape[1] == 128,
                "block_sparse_attention: block_shape only supports [128, 128]");
    (void)inner_precise; (void)num_key_value_heads;
    const bool tnd = q_input_layout == "TND";
    at::Tensor out = at::empty_like(query);
    at::Tensor lse = tnd ? at::empty({query.size(0), query.size(1), 1}, query.options().dtype(at::kFloat))
                         : at::empty({query.size(0), query.size(1), query.size(2), 1}, query.options().dtype(at::kFloat));
    SparseSpec sp;
    if (block_sparse_mask.has_value()) {
        sp.mode = MINDIESD_SPARSE_MASK;
        sp.mask = &block_sparse_mask.value();
    }
    if (tnd) {
        TORCH_CHECK(query.dim() == 3 && key.dim() == 3 && value.dim() == 3, "block_sparse_attention: TND tensors are 3-D");
        const auto lens_q = actual_seq_lengths.value();
        const auto lens_kv = actual_seq_lengths_kv.value();
        const int64_t b = static_cast<int64_t>(lens_q.size());
        TORCH_CHECK(b > 0 && lens_kv.size() == lens_q.size(), "block_sparse_attention: bad actual_seq_lengths");
        for (int64_t i = 0; i < b; ++i)
            TORCH_CHECK(lens_q[i] == lens_q[0] && lens_kv[i] == lens_kv[0],
                        "block_sparse_attention: TND sequences must share one length");
        TORCH_CHECK(lens_q[0] * b == query.size(0) && lens_kv[0] * b == key.size(0),
                    "block_sparse_attention: actual_seq_lengths do not add up to T");
        // [T, N, D] with T = B*S is [B, S, N, D]; the lse layout [T, N] differs from the kernel's
        // [B, N, S], so it goes through a scratch tensor.
        at::Tensor q4 = query.view({b, lens_q[0], query.size(1), query.size(2)});
        at::Tensor k4 = key.view({b, lens_kv[0], key.size(1), key.size(2)});
        at::Tensor v4 = value.view({b, lens_kv[0], value.size(1), value.size(2)});
        at::Tensor o4 = out.view({b, lens_q[0], query.size(1), query.size(2)});
        AttnExtra ex;  // lse [T, N, 1] = [B, S, N]: the kernel writes it through strides
        ex.lse_stride[0] = lens_q[0] * query.size(1);
        ex.lse_stride[1] = 1;
        ex.lse_stride[2] = query.size(1);
        run_attention(q4, k4, v4, o4, softmax_lse_flag != 0 ? lse.data_ptr<float>() : nullptr, false, scale_value, sp, -1,
                      -1, nullptr, nullptr, nullptr, 0, 0, ex);
    } else {
        int64_t sq = -1, skv = -1;
        if (actual_seq_lengths.has_value()) {
            const auto l = actual_seq_lengths.value();
            TORCH_CHECK(static_cast<int64_t>(l.size()) == query.size(0), "block_sparse_attention: bad actual_seq_lengths");
            for (auto x : l) TORCH_CHECK(x == l[0] && x <= query.size(2), "block_sparse_attention: sequences must share one length");
            sq = l[0];
        }
        if (actual_seq_lengths_kv.has_value()) {
            const auto l = actual_seq_lengths_kv.value();
            TORCH_CHECK(static_cast<int64_t>(l.size()) == key.size(0), "block_sparse_attention: bad actual_seq_lengths_kv");
            for (auto x : l) TORCH_CHECK(x == l[0] && x <= key.size(2), "block_sparse_attention: sequences must share one length");
            skv = l[0];
        }
        AttnExtra ex;  // lse is [B, N, S, 1] with S the padded length: rows past the real length stay -inf
        ex.lse_stride[0] = query.size(1) * query.size(2);
        ex.lse_stride[1] = query.size(2);
        ex.lse_stride[2] = 1;
        if (sq >= 0 && sq < query.size(2)) {
            out.zero_();
            if (softmax_lse_flag != 0) lse.fill_(-std::numeric_limits<float>::infinity());
        }
        run_attention(query, key, value, out, softmax_lse_flag != 0 ? lse.data_ptr<float>() : nullptr, true, scale_value,
                      sp, sq, skv, nullptr, nullptr, nullptr, 0, 0, ex);
    }
    return std::make_tuple(out, lse);
}

// ---- rainfusionattention: compacted block lists ------------------------------------------------------
std::tuple<at::Tensor, at::Tensor> rainfusionattention_cuda(
    const at::Tensor& query, const at::Tensor& key, const at::Tensor& value, const at::Tensor& select_idx,
    const at::Tensor& select_num_idx, at::IntArrayRef blockshape, const c10::optional<at::Tensor>& attn_mask,
    c10::OptionalIntArrayRef actual_seq_qlen, c10::OptionalIntArrayRef actual_seq_kvlen,
    const c10::optional<at::Tensor>& block_table, std::string q_input_layout, std::string kv_input_layout,
    int64_t head_num, int64_t mask_type, double scale, int64_t inner_precise, int64_t block_size) {
    TORCH_CHECK(q_input_layout == "TND" || q_input_layout == "BNSD", "q_input_layout only supports 'TND' and 'BNSD' now.");
    TORCH_CHECK(kv_input_layout == "TND" || kv_input_layout == "BNSD", "kv_input_layout only supports 'TND' and 'BNSD' now.");
    TORCH_CHECK(q_input_layout == kv_input_layout, "q_input_layout and kv_input_layout must be consistent.");
    TORCH_CHECK(blockshape.size() == 2 && blockshape[0] == 128 && blockshape[1] == 128,
                "rainfusionattention: blockshape only supports [128, 128]");
    TORCH_CHECK(!attn_mask.has_value() && !block_table.has_value() && mask_type == 0 && block_size == 0,
                "rainfusionattention: attn_mask, block_table, mask_type and block_size are not supported");
    TORCH_CHECK(select_idx.is_cuda() && select_idx.scalar_type() == at::kLong && select_idx.dim() == 3,
                "rainfusionattention: select_idx must be a CUDA int64 tensor [q_blocks, N, kv_blocks]");
    TORCH_CHECK(select_num_idx.is_cuda() && select_num_idx.scalar_type() == at::kLong && select_num_idx.dim() == 2,
                "rainfusionattention: select_num_idx must be a CUDA int64 tensor [q_blocks, N]");
    (void)head_num; (void)inner_precise;
    at::Tensor sel = select_idx.contiguous();
    at::Tensor num = select_num_idx.contiguous();
    at::Tensor out = at::empty_like(query);
    at::Tensor lse = at::empty({query.size(0), query.size(1), query.size(2)}, query.options());
    SparseSpec sp;
    sp.mode = MINDIESD_SPARSE_LIST;
    sp.select_idx = &sel;
    sp.select_num = &num;
    at::Tensor q4, k4, v4, o4;
    bool head_first = true;
    if (q_input_layout == "TND") {
        TORCH_CHECK(query.dim() == 3, "rainfusionattention: TND tensors are 3-D");
        TORCH_CHECK(actual_seq_qlen.has_value() && actual_seq_kvlen.has_value(),
                    "rainfusionattention: actual_seq_qlen and actual_seq_kvlen are required for TND layout.");
        const auto lq = actual_seq_qlen.value();
        const auto lk = actual_seq_kvlen.value();
        const int64_t b = static_cast<int64_t>(lq.size());
        TORCH_CHECK(b > 0 && lk.size() == lq.size(), "rainfusionattention: bad actual_seq_qlen");
        for (int64_t i = 0; i < b; ++i)
            TORCH_CHECK(lq[i] == lq[0] && lk[i] == lk[0], "rainfusionattention: TND sequences must share one length");
        TORCH_CHECK(lq[0] * b == query.size(0) && lk[0] * b == key.size(0), "rainfusionattention: lengths do not add up to T");
        q4 = query.view({b, lq[0], query.size(1), query.size(2)});
        k4 = key.view({b, lk[0], key.size(1), key.size(2)});
        v4 = value.view({b, lk[0], value.size(1), value.size(2)});
        o4 = out.view({b, lq[0], query.size(1), query.size(2)});
        head_first = false;
    } else {
        TORCH_CHECK(query.dim() == 4, "rainfusionattention: BNSD tensors are 4-D");
        q4 = query; k4 = key; v4 = value; o4 = out;
    }
    const int64_t sq = q4.size(head_first ? 2 : 1), skv = k4.size(head_first ? 2 : 1);
    const int64_t heads = q4.size(head_first ? 1 : 2);
    TORCH_CHECK(sel.size(0) == (sq + 127) / 128 && sel.size(1) == heads && sel.size(2) == (skv + 127) / 128,
                "rainfusionattention: select_idx must be [ceil(Sq/128), N, ceil(Skv/128)]");
    TORCH_CHECK(num.size(0) == sel.size(0) && num.size(1) == heads, "rainfusionattention: select_num_idx must be [ceil(Sq/128), N]");
    // The op's lse is returned in the query dtype; the kernel writes fp32 [B, N, S].
    at::Tensor lse32 = at::empty({q4.size(0), heads, sq}, query.options().dtype(at::kFloat));
    run_attention(q4, k4, v4, o4, lse32.data_ptr<float>(), head_first, scale, sp);
    if (head_first) lse.copy_(lse32);
    else lse.copy_(lse32.permute({0, 2, 1}).reshape({query.size(0), query.size(1), 1}).expand_as(lse));
    return std::make_tuple(out, lse);
}

// ---- ada_bsa: cumulative-mass mask estimate and attention over the kept blocks -------------------------
// Views a BNSD / BSND / BSH tensor as 4-D and reports whether heads come first.
at::Tensor view_4d(const at::Tensor& t, const std::string& layout, int64_t heads, bool* head_first, const char* op) {
    if (layout == "BNSD" || layout == "BSND") {
        TORCH_CHECK(t.dim() == 4, op, ": ", layout, " tensors are 4-D");
        *head_first = layout == "BNSD";
        return t;
    }
    TORCH_CHECK(layout == "BSH", op, ": input_layout only supports BNSD, BSND and BSH, got ", layout);
    TORCH_CHECK(t.dim() == 3 && heads > 0 && t.size(2) % heads == 0, op, ": BSH tensors are 3-D with H = N * D");
    *head_first = false;
    return t.view({t.size(0), t.size(1), heads, t.size(2) / heads});
}

std::tuple<at::Tensor, at::Tensor> sparse_block_estimate_cuda(
    const at::Tensor& query, const at::Tensor& key, c10::OptionalIntArrayRef actual_seq_lengths,
    c10::OptionalIntArrayRef actual_seq_lengths_kv, std::string input_layout, int64_t stride, int64_t sparse_size,
    int64_t num_heads, int64_t num_key_value_heads, double scale_value, double threshold, bool causal, bool keep_sink,
    bool keep_recent, double row_sparse) {
    TORCH_CHECK(num_heads != 0, "num_heads must be nonzero.");
    TORCH_CHECK(sparse_size != 0, "sparse_size must be nonzero.");
    TORCH_CHECK(query.is_cuda() && key.is_cuda(), "sparse_block_estimate: query and key must be CUDA tensors");
    TORCH_CHECK(query.scalar_type() == key.scalar_type(), "sparse_block_estimate: query and key must share a dtype");
    TORCH_CHECK(!actual_seq_lengths.has_value() && !actual_seq_lengths_kv.has_value(),
                "sparse_block_estimate: actual_seq_lengths are not supported");
    TORCH_CHECK(stride == 8 && sparse_size == 128, "sparse_block_estimate: only stride=8 and sparse_size=128 are supported");
    bool head_first = true, head_first_k = true;
    at::Tensor q4 = view_4d(query, input_layout, num_heads, &head_first, "sparse_block_estimate");
    at::Tensor k4 = view_4d(key, input_layout, num_key_value_heads, &head_first_k, "sparse_block_estimate");
    const int sdim = head_first ? 2 : 1, ndim = head_first ? 1 : 2;
    const int64_t b = q4.size(0), nq = q4.size(ndim), s = q4.size(sdim), d = q4.size(3);
    TORCH_CHECK(k4.size(0) == b && k4.size(sdim) == s && k4.size(3) == d && nq % k4.size(ndim) == 0,
                "sparse_block_estimate: key must have the query's batch, length and head size");
    // A ragged last group is completed with zero tokens, as the reference's golden does.
    if (s % 8) {
        const int64_t pad = 8 - s % 8;
        std::vector<int64_t> pads = head_first ? std::vector<int64_t>{0, 0, 0, pad} : std::vector<int64_t>{0, 0, 0, 0, 0, pad};
        q4 = at::constant_pad_nd(q4, pads, 0);
        k4 = at::constant_pad_nd(k4, pads, 0);
    }
    const int64_t blocks = (s + sparse_size - 1) / sparse_size;
    const int64_t cols = (blocks + 31) / 32 * 32;
    at::Tensor mask = at::empty({b, nq, blocks, cols}, query.options().dtype(at::kChar));
    at::Tensor count = at::empty({b, nq, blocks}, query.options().dtype(at::kInt));
    mindiesd_estimate_args a = {};
    a.q = q4.data_ptr();
    a.k = k4.data_ptr();
    fill_strides(q4, head_first, a.q_stride);
    fill_strides(k4, head_first, a.k_stride);
    a.dtype = dtype_code(q4.scalar_type());
    a.batch = static_cast<int32_t>(b);
    a.heads = static_cast<int32_t>(nq);
    a.kv_heads = static_cast<int32_t>(k4.size(ndim));
    a.seq = static_cast<int32_t>(q4.size(sdim));
    a.head_dim = static_cast<int32_t>(d);
    a.stride = static_cast<int32_t>(stride);
    a.sparse_size = static_cast<int32_t>(sparse_size);
    a.scale = static_cast<float>(scale_value);
    a.threshold = static_cast<float>(threshold);
    a.row_sparse = row_sparse;
    a.keep_sink = keep_sink;
    a.keep_recent = keep_recent;
    a.causal = causal ? 1 : 0;
    a.causal_key_tokens = static_cast<int32_t>(s);  // the length before the zero completion
    a.mask = mask.data_ptr<int8_t>();
    a.mask_cols = static_cast<int32_t>(cols);
    a.count = count.data_ptr<int32_t>();
    // The kernels size their rows by the padded length; the mask keeps the caller's block count.
    TORCH_CHECK((a.seq + 127) / 128 == blocks, "sparse_block_estimate: internal block count mismatch");
    const size_t bytes = mindiesd_sparse_block_estimate_scratch_bytes(a.batch, a.heads, a.seq);
    at::Tensor scratch = at::empty({static_cast<int64_t>(bytes)}, query.options().dtype(at::kByte));
    a.scratch = scratch.data_ptr();
    a.scratch_bytes = bytes;
    c10::cuda::CUDAGuard guard(query.device());
    check_rc(mindiesd_sparse_block_estimate(&a, stream_of(query)), "mindiesd_sparse_block_estimate");
    return std::make_tuple(mask, count);
}

at::Tensor ada_block_sparse_attention_cuda(const at::Tensor& query, const at::Tensor& key, const at::Tensor& value,
                                           const at::Tensor& sparse_mask, const at::Tensor& sparse_count_table,
                                           std::string input_layout, int64_t sparse_size, int64_t num_heads,
                                           int64_t num_key_value_heads, double scale_value, bool causal,
                                           int64_t inner_precise, int64_t pre_tokens, int64_t next_tokens,
                                           c10::OptionalIntArrayRef actual_seq_lengths,
                                           c10::OptionalIntArrayRef actual_seq_lengths_kv) {
    TORCH_CHECK(sparse_size == 128, "ada_block_sparse_attention: only sparse_size=128 is supported");
    TORCH_CHECK(!actual_seq_lengths.has_value() && !actual_seq_lengths_kv.has_value(),
                "ada_block_sparse_attention: actual_seq_lengths are not supported");
    TORCH_CHECK(sparse_count_table.is_cuda() && sparse_count_table.scalar_type() == at::kInt,
                "ada_block_sparse_attention: sparse_count_table must be a CUDA int32 tensor");
    (void)inner_precise; (void)pre_tokens; (void)next_tokens;
    bool head_first = true, hk = true, hv = true;
    at::Tensor out = at::empty_like(query);
    at::Tensor q4 = view_4d(query, input_layout, num_heads, &head_first, "ada_block_sparse_attention");
    at::Tensor k4 = view_4d(key, input_layout, num_key_value_heads, &hk, "ada_block_sparse_attention");
    at::Tensor v4 = view_4d(value, input_layout, num_key_value_heads, &hv, "ada_block_sparse_attention");
    at::Tensor o4 = out.dim() == 4 ? out : out.view(q4.sizes());
    SparseSpec sp;
    sp.mode = MINDIESD_SPARSE_MASK;
    sp.mask = &sparse_mask;
    AttnExtra ex;
    ex.causal = causal;  // token-level triangle inside the blocks the mask keeps
    run_attention(q4, k4, v4, o4, nullptr, head_first, scale_value, sp, -1, -1, nullptr, nullptr, nullptr, 0, 0, ex);
    return out;
}

// ---- dense attention in the caller's layout ---------------------------------------------------------
at::Tensor attention_fwd_cuda(const at::Tensor& query, const at::Tensor& key, const at::Tensor& value, double scale,
                              bool head_first, bool causal) {
    AttnExtra ex;
    ex.causal = causal;
    if (query.dim() == 4 && query.size(3) != 128) {
        const int64_t d = query.size(3);
        at::Tensor q = pad_head_dim(query), k = pad_head_dim(key), v = pad_head_dim(value);
        at::Tensor wide = at::empty(q.sizes(), q.options());
        run_attention(q, k, v, wide, nullptr, head_first, scale, SparseSpec{}, -1, -1, nullptr, nullptr, nullptr, 0, 0, ex);
        return wide.narrow(3, 0, d).contiguous();
    }
    at::Tensor out = at::empty_like(query);
    if (!out.is_contiguous() && out.stride(3) != 1) out = at::empty(query.sizes(), query.options());
    run_attention(query, key, value, out, nullptr, head_first, scale, SparseSpec{}, -1, -1, nullptr, nullptr, nullptr, 0, 0,
                  ex);
    return out;
}

// ---- RainFusion block-sparse attention on un-permuted tensors ---------------------------------------------
// Mask (or lists) in the block order of the window permutation; the output comes back in the original token
// order without a copy of its own.  inputs_permuted: q, k, v were permuted beforehand (rf_rearrange);
// otherwise they are in their original order and the kernel fetches the permuted order itself.
at::Tensor rf_sparse_attention_cuda(const at::Tensor& query, const at::Tensor& key, const at::Tensor& value,
                                    const c10::optional<at::Tensor>& block_mask,
                                    const c10::optional<at::Tensor>& select_idx,
                                    const c10::optional<at::Tensor>& select_num_idx, at::IntArrayRef latent_shape,
                                    int64_t txt_len, double scale, std::string input_layout, bool inputs_permuted,
                                    const c10::optional<at::Tensor>& q_pairs) {
    TORCH_CHECK(input_layout == "BNSD" || input_layout == "BSND", "rf_sparse_attention: input_layout must be 'BNSD' or 'BSND'");
    TORCH_CHECK(latent_shape.size() == 3, "rf_sparse_attention: latent_shape must be (t, h, w)");
    TORCH_CHECK(inputs_permuted || (latent_shape[2] % 8 == 0 && txt_len % 8 == 0 && txt_len >= 0),
                "rf_sparse_attention: fetching the permuted order inside the kernel needs the grid width and the text "
                "length to be multiples of 8");
    TORCH_CHECK(block_mask.has_value() != (select_idx.has_value() && select_num_idx.has_value()),
                "rf_sparse_attention: pass either block_mask or select_idx and select_num_idx");
    const bool head_first = input_layout == "BNSD";
    at::Tensor out = at::empty(query.sizes(), query.options());
    SparseSpec sp;
    at::Tensor sel, num;
    if (block_mask.has_value()) {
        sp.mode = MINDIESD_SPARSE_MASK;
        sp.mask = &block_mask.value();
    } else {
        sel = select_idx.value().contiguous();
        num = select_num_idx.value().contiguous();
        const int64_t blocks = (query.size(head_first ? 2 : 1) + 127) / 128;
        TORCH_CHECK(sel.is_cuda() && sel.scalar_type() == at::kLong && sel.dim() == 3 && sel.size(0) == blocks &&
                        sel.size(2) == blocks && num.is_cuda() && num.scalar_type() == at::kLong && num.dim() == 2 &&
                        num.size(0) == blocks,
                    "rf_sparse_attention: select_idx must be int64 [blocks, N, blocks], select_num_idx int64 [blocks, N]");
        sp.mode = MINDIESD_SPARSE_LIST;
        sp.select_idx = &sel;
        sp.select_num = &num;
    }
    if (q_pairs.has_value()) {
        TORCH_CHECK(inputs_permuted, "rf_sparse_attention: q_pairs needs q, k, v in the permuted order (inputs_permuted)");
        sp.q_pairs = &q_pairs.value();
    }
    AttnExtra ex;
    ex.perm[0] = static_cast<int>(latent_shape[0]);
    ex.perm[1] = static_cast<int>(latent_shape[1]);
    ex.perm[2] = static_cast<int>(latent_shape[2]);
    ex.perm[3] = static_cast<int>(txt_len);
    ex.perm_inputs_permuted = inputs_permuted;
    run_attention(query, key, value, out, nullptr, head_first, scale, sp, -1, -1, nullptr, nullptr, nullptr, 0, 0, ex);
    return out;
}

// The pairing table of a block mask (mindiesd_rf_pair_blocks), for callers that keep a mask across steps.
at::Tensor rf_pair_blocks_cuda(const at::Tensor& block_mask) {
    TORCH_CHECK(block_mask.is_cuda() && block_mask.scalar_type() == at::kChar && block_mask.dim() == 4 &&
                    block_mask.stride(3) == 1,
                "rf_pair_blocks: block_mask must be a CUDA int8 tensor [B, N, q_blocks, kv_blocks]");
    const int64_t qb = block_mask.size(2);
    at::Tensor pairs = at::empty({block_mask.size(0), block_mask.size(1), (qb + 1) / 2, 2}, block_mask.options().dtype(at::kInt));
    mindiesd_pair_args pa = {};
    pa.mask = block_mask.data_ptr<int8_t>();
    for (int i = 0; i < 3; ++i) pa.mask_stride[i] = block_mask.stride(i);
    pa.batch = static_cast<int32_t>(block_mask.size(0));
    pa.heads = static_cast<int32_t>(block_mask.size(1));
    pa.q_blocks = static_cast<int32_t>(qb);
    pa.kv_blocks = static_cast<int32_t>(block_mask.size(3));
    pa.pairs = pairs.data_ptr<int32_t>();
    c10::cuda::CUDAGuard guard(block_mask.device());
    check_rc(mindiesd_rf_pair_blocks(&pa, stream_of(block_mask)), "mindiesd_rf_pair_blocks");
    return pairs;
}

// ---- packed variable-length sequences (TND): one launch, sequence boundaries read on the device ------------
at::Tensor attention_varlen_fwd_cuda(const at::Tensor& query, const at::Tensor& key, const at::Tensor& value,
                                     const at::Tensor& cu_seqlens_q, const at::Tensor& cu_seqlens_k, double scale,
                                     bool causal) {
    TORCH_CHECK(query.dim() == 3 && key.dim() == 3 && value.dim() == 3, "attention_varlen_fwd: q, k, v are (T, N, D)");
    at::Tensor q = query.stride(2) == 1 ? query : query.contiguous();
    at::Tensor k = key.stride(2) == 1 ? key : key.contiguous();
    at::Tensor v = value.stride(2) == 1 ? value : value.contiguous();
    at::Tensor out = at::empty(q.sizes(), q.options());
    at::Tensor q4 = q.unsqueeze(0), k4 = k.unsqueeze(0), v4 = v.unsqueeze(0), o4 = out.unsqueeze(0);  // [1, T, N, D]
    AttnExtra ex;
    ex.causal = causal;
    ex.cu_seqlens_q = &cu_seqlens_q;
    ex.cu_seqlens_kv = &cu_seqlens_k;
    run_attention(q4, k4, v4, o4, nullptr, false, scale, SparseSpec{}, -1, -1, nullptr, nullptr, nullptr, 0, 0, ex);
    return out;
}

// ---- RainFusion permutation ---------------------------------------------------------------------------
at::Tensor rf_rearrange_cuda(const at::Tensor& x, at::IntArrayRef latent_shape, int64_t txt_len, std::string input_layout,
                             bool inverse) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 4, "rf_rearrange: x must be a 4-D CUDA tensor");
    TORCH_CHECK(input_layout == "BNSD" || input_layout == "BSND", "rf_rearrange: input_layout must be 'BNSD' or 'BSND'");
    TORCH_CHECK(latent_shape.size() == 3, "rf_rearrange: latent_shape must be (t, h, w)");
    const bool head_first = input_layout == "BNSD";
    at::Tensor src = x.stride(3) == 1 ? x : x.contiguous();
    at::Tensor dst = at::empty(src.sizes(), src.options());
    mindiesd_rearrange_args a = {};
    a.src = src.data_ptr();
    a.dst = dst.data_ptr();
    a.batch = static_cast<int32_t>(src.size(0));
    a.heads = static_cast<int32_t>(src.size(head_first ? 1 : 2));
    a.seq = static_cast<int32_t>(src.size(head_first ? 2 : 1));
    a.head_dim = static_cast<int32_t>(src.size(3));
    a.elem_bytes = static_cast<int32_t>(src.element_size());
    fill_strides(src, head_first, a.src_stride);
    fill_strides(dst, head_first, a.dst_stride);
    a.t = static_cast<int32_t>(latent_shape[0]);
    a.h = static_cast<int32_t>(latent_shape[1]);
    a.w = static_cast<int32_t>(latent_shape[2]);
    a.txt_len = static_cast<int32_t>(txt_len);
    a.inverse = inverse ? 1 : 0;
    c10::cuda::CUDAGuard guard(x.device());
    check_rc(mindiesd_rf_rearrange(&a, stream_of(x)), "mindiesd_rf_rearrange");
    return dst;
}

// ---- RainFusion mask builder -----------------------------------------------------------------------------
std::tuple<at::Tensor, at::Tensor, at::Tensor> rf_block_mask_cuda(const at::Tensor& query, const at::Tensor& key,
                                                                  at::IntArrayRef latent_shape, int64_t txt_len,
                                                                  double sparsity, double scale, int64_t block_size,
                                                                  std::string input_layout, bool protect_first_frame,
                                                                  int64_t temporal_band, bool return_lists) {
    TORCH_CHECK(query.is_cuda() && key.is_cuda() && query.dim() == 4 && key.dim() == 4,
                "rf_block_mask: query and key must be 4-D CUDA tensors");
    TORCH_CHECK(query.sizes() == key.sizes() && query.scalar_type() == key.scalar_type(),
                "rf_block_mask: query and key must share shape and dtype");
    TORCH_CHECK(input_layout == "BNSD" || input_layout == "BSND", "rf_block_mask: input_layout must be 'BNSD' or 'BSND'");
    TORCH_CHECK(latent_shape.size() == 3, "rf_block_mask: latent_shape must be (t, h, w)");
    const bool head_first = input_layout == "BNSD";
    at::Tensor q = query.stride(3) == 1 ? query : query.contiguous();
    at::Tensor k = key.stride(3) == 1 ? key : key.contiguous();
    mindiesd_mask_args a = {};
    a.q = q.data_ptr();
    a.k = k.data_ptr();
    a.batch = static_cast<int32_t>(q.size(0));
    a.heads = static_cast<int32_t>(q.size(head_first ? 1 : 2));
    a.seq = static_cast<int32_t>(q.size(head_first ? 2 : 1));
    a.head_dim = static_cast<int32_t>(q.size(3));
    fill_strides(q, head_first, a.q_stride);
    fill_strides(k, head_first, a.k_stride);
    a.dtype = dtype_code(q.scalar_type());
    a.t = static_cast<int32_t>(latent_shape[0]);
    a.h = static_cast<int32_t>(latent_shape[1]);
    a.w = static_cast<int32_t>(latent_shape[2]);
    a.txt_len = static_cast<int32_t>(txt_len);
    a.block_size = static_cast<int32_t>(block_size);
    a.scale = static_cast<float>(scale);
    a.sparsity = sparsity;
    a.protect_first_frame = protect_first_frame ? 1 : 0;
    a.temporal_band = static_cast<int32_t>(temporal_band);
    const int64_t img = static_cast<int64_t>(a.t) * a.h * a.w;
    const int64_t blocks = (img + 127) / 128 + (txt_len + 127) / 128;
    at::Tensor mask = at::empty({a.batch, a.heads, blocks, blocks}, q.options().dtype(at::kChar));
    at::Tensor sel, num;
    a.mask = mask.data_ptr<int8_t>();
    if (return_lists) {
        sel = at::empty({blocks, a.heads, blocks}, q.options().dtype(at::kLong));
        num = at::empty({blocks, a.heads}, q.options().dtype(at::kLong));
        a.select_idx = sel.data_ptr<int64_t>();
        a.select_num = num.data_ptr<int64_t>();
    } else {
        sel = at::empty({0}, q.options().dtype(at::kLong));
        num = at::empty({0}, q.options().dtype(at::kLong));
    }
    const size_t bytes = mindiesd_rf_block_mask_scratch_bytes(a.batch, a.heads, a.seq, a.head_dim);
    at::Tensor scratch = at::empty({static_cast<int64_t>(bytes)}, q.options().dtype(at::kByte));
    a.scratch = scratch.data_ptr();
    a.scratch_bytes = bytes;
    c10::cuda::CUDAGuard guard(q.device());
    check_rc(mindiesd_rf_block_mask(&a, stream_of(q)), "mindiesd_rf_block_mask");
    return std::make_tuple(mask, sel, num);
}

// ---- the two stages of the mask builder on their own -----------------------------------------------------
at::Tensor rf_pool_cuda(const at::Tensor& x, at::IntArrayRef latent_shape, int64_t txt_len, int64_t block_size,
                        std::string input_layout, bool permute) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 4, "rf_pool: x must be a 4-D CUDA tensor");
    TORCH_CHECK(input_layout == "BNSD" || input_layout == "BSND", "rf_pool: input_layout must be 'BNSD' or 'BSND'");
    const bool head_first = input_layout == "BNSD";
    at::Tensor src = x.stride(3) == 1 ? x : x.contiguous();
    mindiesd_pool_args a = {};
    a.x = src.data_ptr();
    a.batch = static_cast<int32_t>(src.size(0));
    a.heads = static_cast<int32_t>(src.size(head_first ? 1 : 2));
    a.seq = static_cast<int32_t>(src.size(head_first ? 2 : 1));
    a.head_dim = static_cast<int32_t>(src.size(3));
    fill_strides(src, head_first, a.x_stride);
    a.dtype = dtype_code(src.scalar_type());
    a.block_size = static_cast<int32_t>(block_size);
    a.permute = permute ? 1 : 0;
    int64_t blocks = (a.seq + 127) / 128;
    if (permute) {
        TORCH_CHECK(latent_shape.size() == 3, "rf_pool: latent_shape must be (t, h, w)");
        a.t = static_cast<int32_t>(latent_shape[0]);
        a.h = static_cast<int32_t>(latent_shape[1]);
        a.w = static_cast<int32_t>(latent_shape[2]);
        a.txt_len = static_cast<int32_t>(txt_len);
        blocks = (static_cast<int64_t>(a.t) * a.h * a.w + 127) / 128 + (txt_len + 127) / 128;
    }
    at::Tensor pooled = at::empty({a.batch, a.heads, blocks, a.head_dim}, src.options().dtype(at::kFloat));
    a.pooled = pooled.data_ptr<float>();
    c10::cuda::CUDAGuard guard(x.device());
    check_rc(mindiesd_rf_pool(&a, stream_of(x)), "mindiesd_rf_pool");
    return pooled;  // [B, N, blocks, D] fp32
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> rf_mask_from_pooled_cuda(const at::Tensor& q_pooled,
                                                                        const at::Tensor& k_pooled,
                                                                        at::IntArrayRef latent_shape, int64_t txt_len,
                                                                        double sparsity, int64_t block_size,
                                                                        bool protect_first_frame, int64_t temporal_band,
                                                                        bool return_lists) {
    TORCH_CHECK(q_pooled.is_cuda() && k_pooled.is_cuda() && q_pooled.dim() == 4 && q_pooled.sizes() == k_pooled.sizes(),
                "rf_mask_from_pooled: pooled q and k must be CUDA tensors [B, N, blocks, D] of one shape");
    TORCH_CHECK(latent_shape.size() == 3, "rf_mask_from_pooled: latent_shape must be (t, h, w)");
    at::Tensor qp = q_pooled.to(at::kFloat).contiguous(), kp = k_pooled.to(at::kFloat).contiguous();
    mindiesd_pooled_mask_args a = {};
    a.q_pooled = qp.data_ptr<float>();
    a.k_pooled = kp.data_ptr<float>();
    a.batch = static_cast<int32_t>(qp.size(0));
    a.heads = static_cast<int32_t>(qp.size(1));
    a.blocks = static_cast<int32_t>(qp.size(2));
    a.head_dim = static_cast<int32_t>(qp.size(3));
    a.t = static_cast<int32_t>(latent_shape[0]);
    a.h = static_cast<int32_t>(latent_shape[1]);
    a.w = static_cast<int32_t>(latent_shape[2]);
    a.txt_len = static_cast<int32_t>(txt_len);
    a.block_size = static_cast<int32_t>(block_size);
    a.protect_first_frame = protect_first_frame ? 1 : 0;
    a.temporal_band = static_cast<int32_t>(temporal_band);
    a.sparsity = sparsity;
    at::Tensor mask = at::empty({a.batch, a.heads, a.blocks, a.blocks}, qp.options().dtype(at::kChar));
    a.mask = mask.data_ptr<int8_t>();
    at::Tensor sel, num;
    if (return_lists) {
        sel = at::empty({a.blocks, a.heads, a.blocks}, qp.options().dtype(at::kLong));
        num = at::empty({a.blocks, a.heads}, qp.options().dtype(at::kLong));
        a.select_idx = sel.data_ptr<int64_t>();
        a.select_num = num.data_ptr<int64_t>();
    } else {
        sel = at::empty({0}, qp.options().dtype(at::kLong));
        num = at::empty({0}, qp.options().dtype(at::kLong));
    }
    c10::cuda::CUDAGuard guard(qp.device());
    check_rc(mindiesd_rf_mask_from_pooled(&a, stream_of(qp)), "mindiesd_rf_mask_from_pooled");
    return std::make_tuple(mask, sel, num);
}

// ---- FP8 quantisation and attention ----------------------------------------------------------------------
std::tuple<at::Tensor, at::Tensor> fa_block_quant_cuda(const at::Tensor& x, int64_t block_size, bool head_first,
                                                       bool per_channel, bool rotate) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 4, "fa_block_quant: x must be a 4-D CUDA tensor");
    at::Tensor src = x.stride(3) == 1 ? x : x.contiguous();
    mindiesd_quant_args a = {};
    a.x = src.data_ptr();
    a.batch = static_cast<int32_t>(src.size(0));
    a.heads = static_cast<int32_t>(src.size(head_first ? 1 : 2));
    a.seq = static_cast<int32_t>(src.size(head_first ? 2 : 1));
    a.head_dim = static_cast<int32_t>(src.size(3));
    fill_strides(src, head_first, a.x_stride);
    a.dtype = dtype_code(src.scalar_type());
    a.mode = per_channel ? 1 : 0;
    a.row_block = static_cast<int32_t>(block_size);
    a.rotate = rotate ? 1 : 0;
    at::Tensor out = at::empty({a.batch, a.heads, a.seq, a.head_dim}, src.options().dtype(at::kFloat8_e4m3fn));
    const int64_t nscale = per_channel ? a.head_dim : (a.seq + block_size - 1) / block_size;
    at::Tensor scales = at::empty({a.batch, a.heads, nscale}, src.options().dtype(at::kFloat));
    a.out = out.data_ptr();
    a.scales = scales.data_ptr<float>();
    c10::cuda::CUDAGuard guard(x.device());
    check_rc(mindiesd_fa_block_quant(&a, stream_of(x)), "mindiesd_fa_block_quant");
    return std::make_tuple(out, scales);
}

std::tuple<at::Tensor, at::Tensor> fa_rotate_quant_cuda(const at::Tensor& x, const at::Tensor& rot, int64_t block_size,
                                                        bool head_first) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 4, "fa_rotate_quant: x must be a 4-D CUDA tensor");
    TORCH_CHECK(rot.is_cuda() && rot.dim() == 2 && rot.size(0) == 128 && rot.size(1) == 128,
                "fa_rotate_quant: rot must be a CUDA tensor [128, 128]");
    at::Tensor src = x.stride(3) == 1 ? x : x.contiguous();
    at::Tensor r = rot.to(src.scalar_type()).contiguous();
    mindiesd_rotate_quant_args a = {};
    a.x = src.data_ptr();
    a.rot = r.data_ptr();
    a.batch = static_cast<int32_t>(src.size(0));
    a.heads = static_cast<int32_t>(src.size(head_first ? 1 : 2));
    a.seq = static_cast<int32_t>(src.size(head_first ? 2 : 1));
    a.head_dim = static_cast<int32_t>(src.size(3));
    fill_strides(src, head_first, a.x_stride);
    a.dtype = dtype_code(src.scalar_type());
    a.row_block = static_cast<int32_t>(block_size);
    at::Tensor out = at::empty({a.batch, a.heads, a.seq, a.head_dim}, src.options().dtype(at::kFloat8_e4m3fn));
    at::Tensor scales = at::empty({a.batch, a.heads, (a.seq + block_size - 1) / block_size}, src.options().dtype(at::kFloat));
    a.out = out.data_ptr();
    a.scales = scales.data_ptr<float>();
    c10::cuda::CUDAGuard guard(x.device());
    check_rc(mindiesd_fa_rotate_quant(&a, stream_of(x)), "mindiesd_fa_rotate_quant");
    return std::make_tuple(out, scales);
}

at::Tensor fp8_attention_cuda(const at::Tensor& query, const at::Tensor& key, const at::Tensor& value,
                              const at::Tensor& q_scale, const at::Tensor& k_scale, const at::Tensor& v_scale,
                              double scale, int64_t k_block, int64_t v_block, at::ScalarType out_dtype) {
    TORCH_CHECK(query.scalar_type() == at::kFloat8_e4m3fn, "fp8_attention: query must be float8_e4m3fn");
    TORCH_CHECK(q_scale.is_cuda() && k_scale.is_cuda() && v_scale.is_cuda() && q_scale.scalar_type() == at::kFloat &&
                    k_scale.scalar_type() == at::kFloat && v_scale.scalar_type() == at::kFloat,
                "fp8_attention: scales must be CUDA fp32 tensors");
    at::Tensor qs = q_scale.contiguous(), ks = k_scale.contiguous(), vs = v_scale.contiguous();
    const int64_t b = query.size(0), n = query.size(1), nkv = key.size(1), sq = query.size(2), skv = key.size(2);
    TORCH_CHECK(qs.numel() == b * n * ((sq + 127) / 128), "fp8_attention: q_scale must hold one value per 128 query tokens");
    TORCH_CHECK(ks.numel() == b * nkv * ((skv + k_block - 1) / k_block), "fp8_attention: k_scale size does not match k_block");
    TORCH_CHECK(vs.numel() == (v_block == 0 ? b * nkv * query.size(3) : b * nkv * ((skv + v_block - 1) / v_block)),
                "fp8_attention: v_scale size does not match v_block");
    at::Tensor out = at::empty(query.sizes(), query.options().dtype(out_dtype));
    run_attention(query, key, value, out, nullptr, true, scale, SparseSpec{}, -1, -1, &qs, &ks, &vs,
                  static_cast<int>(k_block), static_cast<int>(v_block));
    return out;
}

}  // namespace

TORCH_LIBRARY(mindiesd, m) {
    m.def(
        "la(Tensor query, Tensor key, Tensor value, "
        "Tensor? atten_mask=None, Tensor? alibi_mask=None, Tensor? "
        "drop_mask=None, float scale_value=1.0, int head_num=2, str input_layout='BNSD', "
        "float keep_prob=1.0, int pre_tokens=2147483647, int next_tokens=1, "
        "bool is_highPrecision=True)  -> (Tensor, Tensor)");
    m.def(
        "rainfusionattention(Tensor query, Tensor key, Tensor value, Tensor select_idx, "
        "Tensor select_num_idx, int[] blockshape, Tensor? attn_mask=None, int[]? actual_seq_qlen=None, "
        "int[]? actual_seq_kvlen=None, Tensor? block_table=None, str q_input_layout='TND', str kv_input_layout='TND', "
        "int head_num=1, int mask_type=0, float scale=1.0, "
        "int inner_precise=1, int block_size=0) -> (Tensor, Tensor)");
    m.def(
        "block_sparse_attention(Tensor query, Tensor key, Tensor value, "
        "Tensor? block_sparse_mask=None, int[] block_shape=[128,128], "
        "str q_input_layout='BNSD', str kv_input_layout='BNSD', "
        "int num_key_value_heads=1, float scale_value=1.0, int inner_precise=0, "
        "int[]? actual_seq_lengths=None, int[]? actual_seq_lengths_kv=None, "
        "int softmax_lse_flag=0) -> (Tensor, Tensor)");
    m.def(
        "ada_block_sparse_attention(Tensor query, Tensor key, Tensor value, Tensor sparse_mask, Tensor sparse_count_table, "
        "str input_layout='BNSD', int sparse_size=128, int num_heads=1, int num_key_value_heads=1, float scale_value=1, "
        "bool causal=True, int inner_precise=1, int pre_tokens=214748647, int next_tokens=0, "
        "int[]? actual_seq_lengths=None, int[]? actual_seq_lengths_kv=None) -> Tensor");
    m.def(
        "sparse_block_estimate(Tensor query, Tensor key, int[]? actual_seq_lengths=None, "
        "int[]? actual_seq_lengths_kv=None, str input_layout='BNSD', int stride=8, int sparse_size=128, "
        "int num_heads=1, int num_key_value_heads=1, float scale_value=1, float threshold=1, bool causal=True, "
        "bool keep_sink=True, bool keep_recent=True, float row_sparse=1) -> (Tensor, Tensor)");
    // Operators without a counterpart schema in the reference library: there the same steps are
    // torch_npu calls or eager torch code.
    m.def("attention_fwd(Tensor query, Tensor key, Tensor value, float scale, bool head_first, bool causal=False) -> Tensor");
    m.def(
        "rf_sparse_attention(Tensor query, Tensor key, Tensor value, Tensor? block_mask, Tensor? select_idx, "
        "Tensor? select_num_idx, int[] latent_shape, int txt_len, float scale, str input_layout, "
        "bool inputs_permuted=False, Tensor? q_pairs=None) -> Tensor");
    m.def("rf_pair_blocks(Tensor block_mask) -> Tensor");
    m.def(
        "attention_varlen_fwd(Tensor query, Tensor key, Tensor value, Tensor cu_seqlens_q, Tensor cu_seqlens_k, "
        "float scale, bool causal=False) -> Tensor");
    m.def("rf_rearrange(Tensor x, int[] latent_shape, int txt_len, str input_layout, bool inverse) -> Tensor");
    m.def(
        "rf_block_mask(Tensor query, Tensor key, int[] latent_shape, int txt_len, float sparsity, float scale, "
        "int block_size, str input_layout, bool protect_first_frame, int temporal_band, bool return_lists) "
        "-> (Tensor, Tensor, Tensor)");
    m.def("rf_pool(Tensor x, int[] latent_shape, int txt_len, int block_size, str input_layout, bool permute) -> Tensor");
    m.def(
        "rf_mask_from_pooled(Tensor q_pooled, Tensor k_pooled, int[] latent_shape, int txt_len, float sparsity, "
        "int block_size, bool protect_first_frame, int temporal_band, bool return_lists) -> (Tensor, Tensor, Tensor)");
    m.def("fa_block_quant(Tensor x, int block_size, bool head_first, bool per_channel, bool rotate) -> (Tensor, Tensor)");
    m.def("fa_rotate_quant(Tensor x, Tensor rot, int block_size, bool head_first) -> (Tensor, Tensor)");
    m.def(
        "fp8_attention(Tensor query, Tensor key, Tensor value, Tensor q_scale, Tensor k_scale, Tensor v_scale, "
        "float scale, int k_block, int v_block, ScalarType out_dtype) -> Tensor");
}

TORCH_LIBRARY_IMPL(mindiesd, CUDA, m) {
    m.impl("la", &la_cuda);
    m.impl("rainfusionattention", &rainfusionattention_cuda);
    m.impl("block_sparse_attention", &block_sparse_attention_cuda);
    m.impl("ada_block_sparse_attention", &ada_block_sparse_attention_cuda);
    m.impl("sparse_block_estimate", &sparse_block_estimate_cuda);
    m.impl("attention_fwd", &attention_fwd_cuda);
    m.impl("attention_varlen_fwd", &attention_varlen_fwd_cuda);
    m.impl("rf_sparse_attention", &rf_sparse_attention_cuda);
    m.impl("rf_pair_blocks", &rf_pair_blocks_cuda);
    m.impl("rf_rearrange", &rf_rearrange_cuda);
    m.impl("rf_block_mask", &rf_block_mask_cuda);
    m.impl("rf_pool", &rf_pool_cuda);
    m.impl("rf_mask_from_pooled", &rf_mask_from_pooled_cuda);
    m.impl("fa_block_quant", &fa_block_quant_cuda);
    m.impl("fa_rotate_quant", &fa_rotate_quant_cuda);
    m.impl("fp8_attention", &fp8_attention_cuda);
}

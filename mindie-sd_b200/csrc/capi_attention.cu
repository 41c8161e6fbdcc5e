// extern "C" entry points: attention forward, status word, ABI version.
#include "capi_common.h"
#include "fa_fwd.h"
#include "rf_grid.cuh"

#include <mutex>

namespace sdb {

namespace {
__device__ int g_status_word[8];  // [0] code, [1] wait site, [2..4] CTA index of the first report

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
    static EncodeFn fn = [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            sym = nullptr;
        return reinterpret_cast<EncodeFn>(sym);
    }();
    return fn;
}
}  // namespace

int* device_status_word() {
    constexpr int kMaxDevices = 64;
    static std::mutex mu;
    static int* words[kMaxDevices] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!words[dev]) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_status_word) != cudaSuccess) return nullptr;
        words[dev] = static_cast<int*>(ptr);
    }
    return words[dev];
}

namespace {
// Encoded tensor maps, keyed by everything that goes into them.  A denoising loop calls the same
// operator on the same buffers every step (and the pipelined host path once per head chunk), so the
// three driver calls per launch are paid once per buffer.  The map is a pure function of its key;
// the memory behind the pointer may change freely.
struct MapKey {
    const void* base;
    int64_t channels, tokens, heads, batch, stride[3];
    int dtype, box_rows, device;
    bool operator==(const MapKey& o) const {
        return base == o.base && channels == o.channels && tokens == o.tokens && heads == o.heads && batch == o.batch &&
               stride[0] == o.stride[0] && stride[1] == o.stride[1] && stride[2] == o.stride[2] && dtype == o.dtype &&
               box_rows == o.box_rows && device == o.device;
    }
};
constexpr int kMapCacheSize = 128;
struct MapCache {
    std::mutex mu;
    MapKey keys[kMapCacheSize];
    CUtensorMap maps[kMapCacheSize];
    bool used[kMapCacheSize] = {};
    unsigned next = 0;
};
MapCache& map_cache() {
    static MapCache c;
    return c;
}
int encode_tile_map_uncached(CUtensorMap* map, const void* base, int dtype, int64_t channels, int64_t tokens,
                             int64_t heads, int64_t batch, const int64_t stride[3], int box_rows);
}  // namespace

int encode_tile_map(CUtensorMap* map, const void* base, int dtype, int64_t channels, int64_t tokens,
                    int64_t heads, int64_t batch, const int64_t stride[3], int box_rows) {
    MapKey key = {base, channels, tokens, heads, batch, {stride[0], stride[1], stride[2]}, dtype, box_rows, 0};
    if (cudaGetDevice(&key.device) != cudaSuccess) return MINDIESD_E_DRIVER;
    MapCache& c = map_cache();
    {
        std::lock_guard<std::mutex> lock(c.mu);
        for (int i = 0; i < kMapCacheSize; ++i)
            if (c.used[i] && c.keys[i] == key) {
                *map = c.maps[i];
                return MINDIESD_OK;
            }
    }
    const int rc = encode_tile_map_uncached(map, base, dtype, channels, tokens, heads, batch, stride, box_rows);
    if (rc != MINDIESD_OK) return rc;
    std::lock_guard<std::mutex> lock(c.mu);
    const unsigned slot = c.next++ % kMapCacheSize;
    c.keys[slot] = key;
    c.maps[slot] = *map;
    c.used[slot] = true;
    return MINDIESD_OK;
}

namespace {
int encode_tile_map_uncached(CUtensorMap* map, const void* base, int dtype, int64_t channels, int64_t tokens,
                             int64_t heads, int64_t batch, const int64_t stride[3], int box_rows) {
    const int eb = dtype_bytes(dtype);
    if (eb != 1 && eb != 2) return MINDIESD_E_DTYPE;
    EncodeFn fn = encode_fn();
    if (!fn) return MINDIESD_E_DRIVER;
    if (reinterpret_cast<uintptr_t>(base) % 16) return MINDIESD_E_STRIDE;
    for (int i = 0; i < 3; ++i)
        if (stride[i] < 0 || (stride[i] * eb) % 16) return MINDIESD_E_STRIDE;
    const CUtensorMapDataType dt = dtype == MINDIESD_BF16   ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                   : dtype == MINDIESD_FP16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                            : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    // A size-1 dimension may carry any stride; the encoder still wants a multiple of 16 bytes.
    auto bytes = [&](int64_t s, int64_t fallback) { return static_cast<cuuint64_t>((s > 0 ? s : fallback) * eb); };
    const cuuint64_t dims[4] = {static_cast<cuuint64_t>(channels), static_cast<cuuint64_t>(tokens),
                                static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(batch)};
    const cuuint64_t strides[3] = {bytes(stride[2], channels), bytes(stride[1], channels * tokens),
                                   bytes(stride[0], channels * tokens * heads)};
    const cuuint32_t box[4] = {static_cast<cuuint32_t>(128 / eb), static_cast<cuuint32_t>(box_rows), 1, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = fn(map, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? MINDIESD_OK : MINDIESD_E_DRIVER;
}
}  // namespace

}  // namespace sdb

using namespace sdb;

extern "C" int mindiesd_abi_version(void) { return MINDIESD_B200_ABI_VERSION; }

extern "C" int mindiesd_device_status(void) {
    int* w = device_status_word();
    if (!w) return MINDIESD_E_DRIVER;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return static_cast<int>(e);
    int v[8] = {};
    e = cudaMemcpy(v, w, sizeof(v), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (v[0] != 0) {
        const int zero[8] = {};
        cudaMemcpy(w, zero, sizeof(zero), cudaMemcpyHostToDevice);
    }
    return v[0];
}

extern "C" int mindiesd_device_status_detail(int32_t out[8]) {
    int* w = device_status_word();
    if (!w || !out) return MINDIESD_E_NULL;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaMemcpy(out, w, 8 * sizeof(int), cudaMemcpyDeviceToHost);
    return e == cudaSuccess ? MINDIESD_OK : static_cast<int>(e);
}

extern "C" int mindiesd_attention_fwd(const mindiesd_attn_args* a, void* stream) {
    if (!a || !a->q || !a->k || !a->v || !a->out) return MINDIESD_E_NULL;
    if (a->head_dim != 128) return MINDIESD_E_SHAPE;
    if (a->batch <= 0 || a->heads <= 0 || a->kv_heads <= 0 || a->seq_q <= 0 || a->seq_kv <= 0) return MINDIESD_E_SHAPE;
    if (a->heads % a->kv_heads) return MINDIESD_E_SHAPE;
    if (a->batch > 65535 || a->heads > 65535) return MINDIESD_E_SHAPE;
    const bool fp8 = a->in_dtype == MINDIESD_E4M3;
    if (a->in_dtype != MINDIESD_BF16 && a->in_dtype != MINDIESD_FP16 && !fp8) return MINDIESD_E_DTYPE;
    int out_dtype = a->out_dtype;
    if (out_dtype != MINDIESD_BF16 && out_dtype != MINDIESD_FP16 && out_dtype != MINDIESD_FP32) return MINDIESD_E_DTYPE;
    if (!(a->scale > 0.0f) || !(a->scale < 1e30f)) return MINDIESD_E_VALUE;

    FaParams p = {};
    p.q_blocks = (a->seq_q + 127) / 128;
    p.kv_blocks = (a->seq_kv + 127) / 128;
    if (p.kv_blocks > kMaxKvBlocks) return MINDIESD_E_CAPACITY;
    int rc;
    if ((rc = encode_tile_map(&p.tm_q, a->q, a->in_dtype, 128, a->seq_q, a->heads, a->batch, a->q_stride, 128))) return rc;
    if ((rc = encode_tile_map(&p.tm_k, a->k, a->in_dtype, 128, a->seq_kv, a->kv_heads, a->batch, a->k_stride, 128))) return rc;
    if ((rc = encode_tile_map(&p.tm_v, a->v, a->in_dtype, 128, a->seq_kv, a->kv_heads, a->batch, a->v_stride, 128))) return rc;
    const int ob = out_dtype == MINDIESD_FP32 ? 4 : 2;
    if (reinterpret_cast<uintptr_t>(a->out) % 16) return MINDIESD_E_STRIDE;
    for (int i = 0; i < 3; ++i) {
        if (a->o_stride[i] < 0 || (a->o_stride[i] * ob) % 16) return MINDIESD_E_STRIDE;
        p.o_stride[i] = a->o_stride[i];
    }
    p.out = a->out;
    p.lse = a->lse;
    p.batch = a->batch;
    p.heads = a->heads;
    p.kv_heads = a->kv_heads;
    p.seq_q = a->seq_q;
    p.seq_kv = a->seq_kv;
    p.in_dtype = fp8 ? 3 : a->in_dtype;
    p.out_dtype = out_dtype;
    p.scale_log2 = a->scale * 1.4426950408889634f;

    p.sparse_mode = a->sparse_mode;
    if (a->sparse_mode != MINDIESD_SPARSE_NONE) {
        if (a->block_size != 128) return MINDIESD_E_SHAPE;
        if (a->sparse_mode == MINDIESD_SPARSE_MASK) {
            if (!a->block_mask) return MINDIESD_E_NULL;
            p.block_mask = a->block_mask;
            for (int i = 0; i < 3; ++i) p.mask_stride[i] = a->mask_stride[i];
        } else if (a->sparse_mode == MINDIESD_SPARSE_LIST) {
            if (!a->select_idx || !a->select_num) return MINDIESD_E_NULL;
            p.select_idx = a->select_idx;
            p.select_num = a->select_num;
            p.select_stride = p.kv_blocks;
        } else {
            return MINDIESD_E_VALUE;
        }
    }
    if (fp8) {
        if (!a->q_scale || !a->k_scale || !a->v_scale) return MINDIESD_E_NULL;
        auto ok_block = [](int b) { return b == 128 || b == 256 || b == 512; };
        if (!ok_block(a->k_scale_block)) return MINDIESD_E_SHAPE;
        if (a->v_scale_block != 0 && !ok_block(a->v_scale_block)) return MINDIESD_E_SHAPE;
        p.q_scale = a->q_scale;
        p.k_scale = a->k_scale;
        p.v_scale = a->v_scale;
        p.k_scale_block = a->k_scale_block;
        p.k_scale_count = (a->seq_kv + a->k_scale_block - 1) / a->k_scale_block;
        p.v_scale_block = a->v_scale_block;
        p.v_scale_count = a->v_scale_block ? (a->seq_kv + a->v_scale_block - 1) / a->v_scale_block : 128;
    }
    if (a->lse_stride[0] || a->lse_stride[1] || a->lse_stride[2]) {
        for (int i = 0; i < 3; ++i) {
            if (a->lse_stride[i] < 0) return MINDIESD_E_STRIDE;
            p.lse_stride[i] = a->lse_stride[i];
        }
    } else {
        p.lse_stride[0] = static_cast<int64_t>(a->heads) * a->seq_q;
        p.lse_stride[1] = a->seq_q;
        p.lse_stride[2] = 1;
    }
    p.causal = a->causal != 0;
    if (a->num_seqs < 0) return MINDIESD_E_VALUE;
    if (a->num_seqs > 0) {
        if (!a->cu_seqlens_q || !a->cu_seqlens_kv) return MINDIESD_E_NULL;
        if (a->batch != 1) return MINDIESD_E_SHAPE;
        if (fp8 || a->sparse_mode != MINDIESD_SPARSE_NONE) return MINDIESD_E_VALUE;
        if (a->seq_q / 256 + static_cast<int64_t>(a->num_seqs) > 0x7fffffff) return MINDIESD_E_CAPACITY;
        p.cu_seqlens_q = a->cu_seqlens_q;
        p.cu_seqlens_kv = a->cu_seqlens_kv;
        p.num_seqs = a->num_seqs;
    }
    if (a->perm_t != 0) {
        if (a->perm_t < 0 || a->perm_h <= 0 || a->perm_w <= 0 || a->perm_txt < 0) return MINDIESD_E_SHAPE;
        const Grid g = make_grid(a->perm_t, a->perm_h, a->perm_w, a->perm_txt);
        if (a->seq_q != g.img + g.txt) return MINDIESD_E_SHAPE;
        if (a->num_seqs > 0) return MINDIESD_E_VALUE;
        if (a->perm_inputs_permuted) {
            p.perm_on = 2;
        } else {
            if (!groups_of_eight_are_contiguous(g) || a->seq_kv != a->seq_q) return MINDIESD_E_SHAPE;
            if (fp8) return MINDIESD_E_VALUE;
            if ((rc = encode_tile_map(&p.tm_q8, a->q, a->in_dtype, 128, a->seq_q, a->heads, a->batch, a->q_stride, 8))) return rc;
            if ((rc = encode_tile_map(&p.tm_k8, a->k, a->in_dtype, 128, a->seq_kv, a->kv_heads, a->batch, a->k_stride, 8))) return rc;
            if ((rc = encode_tile_map(&p.tm_v8, a->v, a->in_dtype, 128, a->seq_kv, a->kv_heads, a->batch, a->v_stride, 8))) return rc;
            p.perm_on = 1;
        }
        p.perm_t = a->perm_t;
        p.perm_h = a->perm_h;
        p.perm_w = a->perm_w;
        p.perm_txt = a->perm_txt;
    }
    if (a->q_pairs) {
        if (a->sparse_mode == MINDIESD_SPARSE_NONE || fp8 || a->causal || a->num_seqs > 0 || p.perm_on == 1)
            return MINDIESD_E_VALUE;
        if (a->q_pair_count != (p.q_blocks + 1) / 2) return MINDIESD_E_SHAPE;
        if (reinterpret_cast<uintptr_t>(a->q_pairs) % 4) return MINDIESD_E_STRIDE;
        p.q_pairs = a->q_pairs;
        p.q_pair_count = a->q_pair_count;
    }
    p.wait_limit_us = a->wait_limit_us ? a->wait_limit_us : kDefaultWaitLimitUs;
    p.test_withhold = a->test_withhold;
    p.status = device_status_word();
    const cudaError_t e = fa_fwd_launch(p, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? MINDIESD_OK : static_cast<int>(e);
}

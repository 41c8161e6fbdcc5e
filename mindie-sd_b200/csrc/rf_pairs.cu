// Pairs the 128-row query blocks of a block mask for the block-sparse attention kernel.
//
// A thread block of that kernel works on two query blocks at once and walks the union of their key-block
// lists: a step in which only one of the two wants the key block costs as much as one that serves both.
// Neighbouring query blocks of a RainFusion mask share about four fifths of their lists; choosing the partner
// by overlap instead halves the steps that serve one tile only.
//
// One thread block per (head, batch).  The mask rows become bitmaps in shared memory; the rows are ranked by
// their number of kept blocks (heaviest first, ties by index), and in that order every row still free takes
// the free row with the largest Jaccard overlap |A and B| / |A or B| (compared exactly, as cross products).
#include "capi_common.h"

namespace sdb {

namespace {

constexpr int kMaxBlocks = 1024;             // query and key blocks per head
constexpr int kPairThreads = 512;

struct PairParams {
    const int8_t* mask;
    int64_t stride[3];
    int heads, q_blocks, kv_blocks;
    int32_t* pairs;
};

__global__ void __launch_bounds__(kPairThreads) rf_pair_kernel(const PairParams p) {
    extern __shared__ uint32_t sm[];
    const int words = (p.kv_blocks + 31) / 32;
    uint32_t* bits = sm;                                         // [q_blocks][words]
    int* count = reinterpret_cast<int*>(bits + p.q_blocks * words);  // [q_blocks] kept blocks of a row
    int* order = count + p.q_blocks;                             // [q_blocks] rows, heaviest first
    int* free_row = order + p.q_blocks;                          // [q_blocks] 1 while unpaired
    constexpr int kWarps = kPairThreads / 32;
    __shared__ unsigned long long best[2][kWarps];               // per warp, double-buffered over the steps
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int head = blockIdx.x, batch = blockIdx.y;
    const int8_t* m = p.mask + batch * p.stride[0] + head * p.stride[1];

    // bitmaps: one warp per row, 32 consecutive mask bytes per load, one ballot per word
    for (int r = warp; r < p.q_blocks; r += kWarps) {
        const int8_t* row = m + r * p.stride[2];
        int c = 0;
        for (int w = 0; w < words; ++w) {
            const int j = w * 32 + lane;
            const uint32_t v = __ballot_sync(0xffffffffu, j < p.kv_blocks && row[j] != 0);
            if (lane == 0) bits[r * words + w] = v;
            c += __popc(v);
        }
        if (lane == 0) {
            count[r] = c;
            free_row[r] = 1;
        }
    }
    __syncthreads();
    // rank of every row: rows with more kept blocks first, ties by index
    for (int r = tid; r < p.q_blocks; r += kPairThreads) {
        int rank = 0;
        const int c = count[r];
        for (int o = 0; o < p.q_blocks; ++o) rank += (count[o] > c) || (count[o] == c && o < r);
        order[rank] = r;
    }
    __syncthreads();

    int32_t* out = p.pairs + (static_cast<int64_t>(batch) * p.heads + head) * ((p.q_blocks + 1) / 2) * 2;
    int made = 0;
    for (int k = 0; k < p.q_blocks; ++k) {
        const int a = order[k];
        if (!free_row[a]) continue;  // uniform: every thread wrote the same updates itself
        // key of a candidate: Jaccard overlap inter / (ca + cb - inter) as the bits of a non-negative float
        // (they order like the floats), then the lower index; bit 63 marks "there is a candidate"
        unsigned long long mine = 0;
        const int ca = count[a];
        const uint32_t* ra = bits + a * words;
        for (int b = tid; b < p.q_blocks; b += kPairThreads) {
            if (b == a || !free_row[b]) continue;
            const uint32_t* rb = bits + b * words;
            int inter = 0;
            for (int w = 0; w < words; ++w) inter += __popc(ra[w] & rb[w]);
            const int uni = ca + count[b] - inter;
            const float frac = uni > 0 ? __fdividef(static_cast<float>(inter), static_cast<float>(uni)) : 0.0f;
            const unsigned long long key = (static_cast<unsigned long long>(__float_as_uint(frac)) << 31) |
                                           static_cast<unsigned>(0x7fffffff - b) | (1ull << 63);
            mine = key > mine ? key : mine;
        }
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, mine, o);
            mine = other > mine ? other : mine;
        }
        const int buf = made & 1;
        if (lane == 0) best[buf][warp] = mine;
        __syncthreads();
        // every thread reduces the warps' candidates by itself: one barrier per step
        unsigned long long top = 0;
        for (int w = 0; w < kWarps; ++w) top = best[buf][w] > top ? best[buf][w] : top;
        const int b = top ? 0x7fffffff - static_cast<int>(top & 0x7fffffffu) : -1;
        if (tid == 0) {
            out[2 * made] = a;
            out[2 * made + 1] = b;
        }
        // The rows leave the free list.  Every thread came to the same (a, b) and writes the same two zeros, and
        // a thread reads the list after its own writes: no second barrier is needed (the candidates' buffer
        // alternates, so a thread that runs ahead does not overwrite what a slower one still reads).
        free_row[a] = 0;
        if (b >= 0) free_row[b] = 0;
        ++made;
    }
}

}  // namespace
}  // namespace sdb

using namespace sdb;

extern "C" int mindiesd_rf_pair_blocks(const mindiesd_pair_args* a, void* stream) {
    if (!a || !a->mask || !a->pairs) return MINDIESD_E_NULL;
    if (a->batch <= 0 || a->heads <= 0 || a->q_blocks <= 0 || a->kv_blocks <= 0) return MINDIESD_E_SHAPE;
    if (a->q_blocks > kMaxBlocks || a->kv_blocks > kMaxBlocks) return MINDIESD_E_CAPACITY;
    if (a->batch > 65535) return MINDIESD_E_SHAPE;
    for (int i = 0; i < 3; ++i)
        if (a->mask_stride[i] < 0) return MINDIESD_E_STRIDE;
    if (reinterpret_cast<uintptr_t>(a->pairs) % 4) return MINDIESD_E_STRIDE;
    PairParams p;
    p.mask = a->mask;
    for (int i = 0; i < 3; ++i) p.stride[i] = a->mask_stride[i];
    p.heads = a->heads;
    p.q_blocks = a->q_blocks;
    p.kv_blocks = a->kv_blocks;
    p.pairs = a->pairs;
    const int words = (a->kv_blocks + 31) / 32;
    const size_t smem = (static_cast<size_t>(a->q_blocks) * words + 3 * static_cast<size_t>(a->q_blocks)) * 4;
    cudaError_t e = cudaFuncSetAttribute(rf_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    rf_pair_kernel<<<dim3(a->heads, a->batch), kPairThreads, smem, static_cast<cudaStream_t>(stream)>>>(p);
    e = cudaGetLastError();
    return e == cudaSuccess ? MINDIESD_OK : static_cast<int>(e);
}

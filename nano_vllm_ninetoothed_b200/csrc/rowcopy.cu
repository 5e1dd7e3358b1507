// Indexed row movers: store_kvcache (scatter by slot) and embedding (gather by id).
// Both are pure byte copies, HBM-bound: one warp moves one row with 128-bit
// coalesced accesses, four independent loads in flight per lane before any store.
#include "common.cuh"

namespace b200mops {
namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kUnroll = 4;

// Copy `chunks` 16-byte packets from src to dst with the 32 lanes of one warp.
__device__ __forceinline__ void warp_copy16(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                            int chunks, int lane) {
    int c = lane;
    for (; c + 32 * (kUnroll - 1) < chunks; c += 32 * kUnroll) {
        uint4 r[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const uint4* p = src + c + 32 * u;
            asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(r[u].x), "=r"(r[u].y), "=r"(r[u].z), "=r"(r[u].w) : "l"(p));
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) dst[c + 32 * u] = r[u];
    }
    for (; c < chunks; c += 32) dst[c] = src[c];
}

// Fallback for rows that are not 16-byte aligned: element-wise, still coalesced.
template <typename E>
__device__ __forceinline__ void warp_copy_elems(const E* __restrict__ src, E* __restrict__ dst,
                                                int64_t n, int lane) {
    for (int64_t c = lane; c < n; c += 32) dst[c] = src[c];
}

template <typename E>
__device__ __forceinline__ void warp_zero_elems(E* __restrict__ dst, int64_t n, int lane) {
    for (int64_t c = lane; c < n; c += 32) dst[c] = E(0);
}

// items = 2 * n_tokens: item 2i moves key row i, item 2i+1 moves value row i, so the two
// warps that share a slot lookup sit next to each other.
template <bool kVec16>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
store_kvcache_kernel(const char* __restrict__ key, const char* __restrict__ value,
                     int64_t key_stride_bytes, int64_t value_stride_bytes,
                     char* __restrict__ k_cache, char* __restrict__ v_cache,
                     int64_t slot_stride_bytes, const int32_t* __restrict__ slot_mapping,
                     int64_t n_tokens, int64_t row_bytes, int64_t num_slots,
                     int32_t* __restrict__ status_word) {
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (item >= 2 * n_tokens) return;
    const int64_t tok = item >> 1;
    const bool is_v = item & 1;
    const int32_t slot = __ldg(slot_mapping + tok);
    if (slot == -1) return;
    if (slot < 0 || slot >= num_slots) {
        if (lane == 0 && status_word) atomicOr(status_word, B200MOPS_DEV_BAD_SLOT);
        return;
    }
    const char* src = is_v ? value + tok * value_stride_bytes : key + tok * key_stride_bytes;
    char* dst = (is_v ? v_cache : k_cache) + (int64_t)slot * slot_stride_bytes;
    if (kVec16) {
        warp_copy16(reinterpret_cast<const uint4*>(src), reinterpret_cast<uint4*>(dst),
                    (int)(row_bytes >> 4), lane);
    } else {
        warp_copy_elems(reinterpret_cast<const uint16_t*>(src), reinterpret_cast<uint16_t*>(dst),
                        row_bytes >> 1, lane);
    }
}

template <bool kVec16>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
embedding_kernel(const int64_t* __restrict__ ids, int64_t n_ids,
                 const char* __restrict__ weight, int64_t vocab, int64_t weight_stride_bytes,
                 char* __restrict__ out, int64_t row_bytes, int32_t* __restrict__ status_word) {
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (item >= n_ids) return;
    const int64_t id = __ldg(ids + item);
    char* dst = out + item * row_bytes;
    if (id < 0 || id >= vocab) {
        if (lane == 0 && status_word) atomicOr(status_word, B200MOPS_DEV_BAD_TOKEN_ID);
        warp_zero_elems(reinterpret_cast<uint16_t*>(dst), row_bytes >> 1, lane);
        return;
    }
    const char* src = weight + id * weight_stride_bytes;
    if (kVec16) {
        warp_copy16(reinterpret_cast<const uint4*>(src), reinterpret_cast<uint4*>(dst),
                    (int)(row_bytes >> 4), lane);
    } else {
        warp_copy_elems(reinterpret_cast<const uint16_t*>(src), reinterpret_cast<uint16_t*>(dst),
                        row_bytes >> 1, lane);
    }
}

}  // namespace
}  // namespace b200mops

using namespace b200mops;

extern "C" int b200mops_store_kvcache(const void* key, const void* value,
                                      int64_t key_stride0, int64_t value_stride0,
                                      void* k_cache, void* v_cache, int64_t cache_slot_stride,
                                      const int32_t* slot_mapping, int64_t n_tokens,
                                      int64_t row_elems, int64_t num_slots,
                                      int dtype, int32_t* status_word, void* stream) {
    const int es = dtype_size(dtype);
    if (es == 0) return B200MOPS_ERR_DTYPE;
    if (n_tokens < 0 || row_elems <= 0 || num_slots < 0) return B200MOPS_ERR_SHAPE;
    if (n_tokens == 0) return B200MOPS_OK;
    if (!key || !value || !k_cache || !v_cache || !slot_mapping) return B200MOPS_ERR_NULL_POINTER;
    // The reference asserts the same contract: rows are dense, caches hold one row per slot.
    if (cache_slot_stride < row_elems || key_stride0 < 0 || value_stride0 < 0)
        return B200MOPS_ERR_STRIDE;
    if (2 * n_tokens > (int64_t)INT32_MAX * kWarpsPerBlock) return B200MOPS_ERR_TOO_LARGE;
    const int64_t row_bytes = row_elems * es;
    const int64_t ks = key_stride0 * es, vs = value_stride0 * es, ss = cache_slot_stride * es;
    const bool vec = aligned16(key) && aligned16(value) && aligned16(k_cache) && aligned16(v_cache) &&
                     (row_bytes % 16 == 0) && (ks % 16 == 0) && (vs % 16 == 0) && (ss % 16 == 0);
    const unsigned blocks = (unsigned)((2 * n_tokens + kWarpsPerBlock - 1) / kWarpsPerBlock);
    auto launch = [&](auto kernel) {
        kernel<<<blocks, kWarpsPerBlock * 32, 0, as_stream(stream)>>>(
            (const char*)key, (const char*)value, ks, vs, (char*)k_cache, (char*)v_cache, ss,
            slot_mapping, n_tokens, row_bytes, num_slots, status_word);
    };
    if (vec) launch(store_kvcache_kernel<true>);
    else if (row_bytes % 2 == 0) launch(store_kvcache_kernel<false>);
    else return B200MOPS_ERR_ALIGNMENT;
    return launch_status();
}

extern "C" int b200mops_embedding(const int64_t* ids, int64_t n_ids,
                                  const void* weight, int64_t vocab, int64_t hidden,
                                  int64_t weight_stride0, void* out,
                                  int dtype, int32_t* status_word, void* stream) {
    const int es = dtype_size(dtype);
    if (es == 0) return B200MOPS_ERR_DTYPE;
    if (n_ids < 0 || vocab <= 0 || hidden <= 0) return B200MOPS_ERR_SHAPE;
    if (n_ids == 0) return B200MOPS_OK;
    if (!ids || !weight || !out) return B200MOPS_ERR_NULL_POINTER;
    if (weight_stride0 < hidden) return B200MOPS_ERR_STRIDE;
    if (n_ids > (int64_t)INT32_MAX * kWarpsPerBlock) return B200MOPS_ERR_TOO_LARGE;
    const int64_t row_bytes = hidden * es, ws = weight_stride0 * es;
    const bool vec = aligned16(weight) && aligned16(out) && (row_bytes % 16 == 0) && (ws % 16 == 0);
    const unsigned blocks = (unsigned)((n_ids + kWarpsPerBlock - 1) / kWarpsPerBlock);
    auto launch = [&](auto kernel) {
        kernel<<<blocks, kWarpsPerBlock * 32, 0, as_stream(stream)>>>(
            ids, n_ids, (const char*)weight, vocab, ws, (char*)out, row_bytes, status_word);
    };
    if (vec) launch(embedding_kernel<true>);
    else launch(embedding_kernel<false>);
    return launch_status();
}

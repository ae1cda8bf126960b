// Embedding gather: residual[t, :] = table[ids[t], :], written in 32-bit.
//
// Reference op: row gather with an out-of-vocabulary error
// (backends/cpu/src/backend.rs:282-298). Here the host rejects bad ids before
// the launch; a bad id that still reaches the device writes zeros and sets
// kStatusBadToken in the status word.
#include "common.cuh"

namespace {

template <typename TW>
__global__ void embedding_kernel(const TW* __restrict__ table, const int* __restrict__ ids,
                                 float* __restrict__ out, int hidden, int vocab, float scale,
                                 int* __restrict__ status) {
    qi::pdl_enter();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* dst = out + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0 && status) atomicOr(status, qi::kStatusBadToken);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = 0.f;
        return;
    }
    const TW* src = table + (size_t)id * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = qi::to_f32<TW>(src[i]) * scale;
}

}  // namespace

// residual[t, :] = table[ids[t], :] * scale (the product in 32-bit).
extern "C" int qi_embedding_scaled(const void* table, int table_dtype, const int* ids, float* out,
                                   int n_tokens, int hidden, int vocab, float scale, int* status,
                                   cudaStream_t stream) {
    QI_REQUIRE(n_tokens >= 0 && hidden > 0 && vocab > 0, "embedding: bad sizes n=%d hidden=%d vocab=%d",
               n_tokens, hidden, vocab);
    if (n_tokens == 0) return 0;
    const int threads = hidden >= 1024 ? 256 : (hidden >= 256 ? 128 : 64);
    QI_DISPATCH_DTYPE(table_dtype, TW, {
        qi::launch(embedding_kernel<TW>, dim3(n_tokens), dim3(threads), 0, stream, (const TW*)table, ids, out, hidden, vocab,
                   scale, status);
    });
    return qi::check_launch("embedding");
}

extern "C" int qi_embedding(const void* table, int table_dtype, const int* ids, float* out,
                            int n_tokens, int hidden, int vocab, int* status,
                            cudaStream_t stream) {
    return qi_embedding_scaled(table, table_dtype, ids, out, n_tokens, hidden, vocab, 1.0f, status, stream);
}

// Embedding with a hashed bigram table added: residual[t, :] = table[id_t, :] + bigram[row_t, :], where
//     row_t = (id_(t-1) * mul_prev + id_t * mul_cur) mod buckets      for a token that has a predecessor,
//     row_t = buckets (the table's last row)                          for the first token of a sequence.
// The predecessor of an entry's first token is the last token of the request's previous step, kept in
// `prev_state[slot * state_stride]` (int32, one word a slot). The block of an entry's first token reads that word and
// then writes the entry's last token into it; no other block touches it, so a step needs no second pass.
namespace {

template <typename TW>
__global__ void embedding_bigram_kernel(const TW* __restrict__ table, const TW* __restrict__ bigram,
                                        const int* __restrict__ ids, const int* __restrict__ positions,
                                        const int* __restrict__ token_req, const int* __restrict__ q_start,
                                        const int* __restrict__ slot_ids, int* __restrict__ prev_state,
                                        float* __restrict__ out, int hidden, int vocab, long long buckets,
                                        long long mul_prev, long long mul_cur, long long state_stride,
                                        int* __restrict__ status) {
    __shared__ long long s_row;
    qi::pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    if (threadIdx.x == 0) {
        const int e = token_req[t];
        const int first = q_start[e], last = q_start[e + 1] - 1;
        long long row = buckets;
        if (positions[t] > 0) {
            const long long prev = t > first ? ids[t - 1] : prev_state[(size_t)slot_ids[e] * state_stride];
            row = (prev * mul_prev + (long long)id * mul_cur) % buckets;
            if (row < 0) row += buckets;
        }
        if (t == first) prev_state[(size_t)slot_ids[e] * state_stride] = ids[last];
        s_row = row;
    }
    __syncthreads();
    float* dst = out + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0 && status) atomicOr(status, qi::kStatusBadToken);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = 0.f;
        return;
    }
    const TW* src = table + (size_t)id * hidden;
    const TW* add = bigram + (size_t)s_row * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = qi::to_f32<TW>(src[i]) + qi::to_f32<TW>(add[i]);
}

}  // namespace

extern "C" int qi_embedding_bigram(const void* table, const void* bigram, int table_dtype, const int* ids,
                                   const int* positions, const int* token_req, const int* q_start,
                                   const int* slot_ids, int* prev_state, float* out, int n_tokens, int hidden,
                                   int vocab, long long buckets, long long mul_prev, long long mul_cur,
                                   long long state_stride, int* status, cudaStream_t stream) {
    QI_REQUIRE(state_stride >= 1, "embedding_bigram: the state's slot stride must be at least one word");
    QI_REQUIRE(n_tokens >= 0 && hidden > 0 && vocab > 0 && buckets > 0, "embedding_bigram: bad sizes n=%d hidden=%d vocab=%d buckets=%lld",
               n_tokens, hidden, vocab, buckets);
    QI_REQUIRE(mul_prev >= 0 && mul_cur >= 0 && mul_prev < (1ll << 31) && mul_cur < (1ll << 31), "embedding_bigram: multipliers must fit 31 bits");
    if (n_tokens == 0) return 0;
    const int threads = hidden >= 1024 ? 256 : (hidden >= 256 ? 128 : 64);
    QI_DISPATCH_DTYPE(table_dtype, TW, {
        qi::launch(embedding_bigram_kernel<TW>, dim3(n_tokens), dim3(threads), 0, stream, (const TW*)table, (const TW*)bigram, ids,
                   positions, token_req, q_start, slot_ids, prev_state, out, hidden, vocab, buckets, mul_prev, mul_cur, state_stride, status);
    });
    return qi::check_launch("embedding_bigram");
}

// A bank of short causal convolutions over time, one filter of `taps` weights per channel, with the
// sequence's last taps - 1 inputs kept as state of fixed size between steps:
//
//     out_k[t, c] = (residual ? h[t, c] : 0) + sum_j w_k[j, c] * h[t - taps + 1 + j, c],     j = 0 .. taps - 1
//
// where h[s] for s before the step's first token comes from the request's state (the inputs of its
// earlier steps) and is zero before the sequence's start. Up to two filters read the same input in one
// launch (a layer whose sublayers each have their own filter over one normalised stream), and the
// input can be written once more in the output type (for a consumer that reads it unfiltered).
//
// A bias per channel may be added and silu applied to the sum (`act` 1), as the input convolution of a
// recurrent layer wants; the input may then be a block of columns inside wider rows (`ldh` elements a row)
// in the activation type.
// The state and all sums are 32-bit; inputs 32-bit or the activation type; outputs in the activation type. Weights are laid out
// [filter][tap][channel] so that a warp's loads are contiguous.
//
// One thread per token and one or four neighbouring channels. A token that stands at least taps - 1 places into its entry reads
// only the step's own rows. The thread of an entry's FIRST token also computes the entry's next
// taps - 2 tokens (the only ones that read the old state) and then writes the new state; the threads
// of those tokens do nothing. So the old state is read and the new one written by the same thread, in
// program order, and one launch serves a step of any mix of portions and single tokens.
#include "common.cuh"

namespace {

constexpr int kMaxTaps = 16;

__device__ __forceinline__ float conv_finish(float a, const float* bias, int c, int act) {
    if (bias) a += bias[c];
    return act == 1 ? a / (1.0f + expf(-a)) : a;
}

// VEC neighbouring channels of a row as one access (16 bytes of 32-bit numbers, 8 of bfloat16).
template <typename T, int VEC>
struct alignas(sizeof(T) * VEC) ConvPack {
    T v[VEC];
};

template <typename T, int VEC>
__device__ __forceinline__ void conv_load(const T* p, float (&x)[VEC]) {
    const ConvPack<T, VEC> pk = *reinterpret_cast<const ConvPack<T, VEC>*>(p);
#pragma unroll
    for (int v = 0; v < VEC; ++v) x[v] = qi::to_f32<T>(pk.v[v]);
}

template <typename T, int VEC>
__device__ __forceinline__ void conv_store(T* p, const float (&x)[VEC]) {
    ConvPack<T, VEC> pk;
#pragma unroll
    for (int v = 0; v < VEC; ++v) pk.v[v] = qi::from_f32<T>(x[v]);
    *reinterpret_cast<ConvPack<T, VEC>*>(p) = pk;
}

// The thread of an entry's first token, for channel c: the old state in registers, the entry's first taps - 1 rows (the
// only ones that read it), then the new state.
template <typename TI, typename TO>
__device__ __forceinline__ void conv_entry_head(const TI* __restrict__ h, long long ldh, const float* __restrict__ bias, int act,
                                                const float* __restrict__ w, float* __restrict__ state, TO* __restrict__ out0,
                                                TO* __restrict__ out1, const int* __restrict__ q_start,
                                                const int* __restrict__ start_pos, const int* __restrict__ slot_ids, int e, int first,
                                                int c, int C, int taps, int n_filters, int residual, long long state_stride) {
    const int back = taps - 1;
    const float* w1 = w + (size_t)taps * C;
    const int len = q_start[e + 1] - first;
    const int p0 = start_pos[e];
    float* st = state + (size_t)slot_ids[e] * state_stride + c;
    float old[kMaxTaps];
#pragma unroll
    for (int k = 0; k < kMaxTaps; ++k) old[k] = 0.f;
    for (int k = 0; k < back; ++k) old[k] = (p0 - back + k >= 0) ? st[(size_t)k * C] : 0.f;
    const int head = len < back ? len : back;
    for (int ii = 0; ii < head; ++ii) {
        const float xi = qi::to_f32<TI>(h[(size_t)(first + ii) * ldh + c]);
        float a0 = residual ? xi : 0.f, a1 = a0;
        for (int j = 0; j < taps; ++j) {
            const int rel = ii - back + j;      // place in the entry; negative: in the old state
            float v;
            if (rel >= 0) {
                v = qi::to_f32<TI>(h[(size_t)(first + rel) * ldh + c]);
            } else {
                v = 0.f;
#pragma unroll
                for (int k = 0; k < kMaxTaps; ++k) if (k == back + rel) v = old[k];
            }
            a0 = fmaf(w[(size_t)j * C + c], v, a0);
            if (n_filters > 1) a1 = fmaf(w1[(size_t)j * C + c], v, a1);
        }
        out0[(size_t)(first + ii) * C + c] = qi::from_f32<TO>(conv_finish(a0, bias, c, act));
        if (n_filters > 1) out1[(size_t)(first + ii) * C + c] = qi::from_f32<TO>(conv_finish(a1, bias ? bias + C : nullptr, c, act));
    }
    for (int k = 0; k < back; ++k) {
        const int rel = len - back + k;
        float v;
        if (rel >= 0) {
            v = qi::to_f32<TI>(h[(size_t)(first + rel) * ldh + c]);
        } else {
            v = 0.f;
#pragma unroll
            for (int kk = 0; kk < kMaxTaps; ++kk) if (kk == back + rel) v = old[kk];
        }
        st[(size_t)k * C] = v;
    }
}

// One thread per token and VEC neighbouring channels (VEC 4 where the rows' lengths and addresses allow 16-byte accesses).
template <typename TI, typename TO, int VEC>
__global__ void __launch_bounds__(256)
short_conv_kernel(const TI* __restrict__ h, long long ldh, const float* __restrict__ bias, int act,
                  const float* __restrict__ w, float* __restrict__ state,
                  TO* __restrict__ out0, TO* __restrict__ out1, TO* __restrict__ copy,
                  const int* __restrict__ token_req, const int* __restrict__ q_start,
                  const int* __restrict__ start_pos, const int* __restrict__ slot_ids, int n_tokens, int C,
                  int taps, int n_filters, int residual, long long state_stride) {
    qi::pdl_wait();
    const int CV = C / VEC;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n_tokens * CV) return;
    const int t = (int)(idx / CV), c = (int)(idx % CV) * VEC;
    const int e = token_req[t];
    const int first = q_start[e];
    const int i = t - first;
    float x[VEC];
    conv_load<TI, VEC>(h + (size_t)t * ldh + c, x);
    if (copy) conv_store<TO, VEC>(copy + (size_t)t * C + c, x);
    const int back = taps - 1;
    if (i >= back) {
        const float* w1 = w + (size_t)taps * C;
        float a0[VEC], a1[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) a0[v] = a1[v] = residual ? x[v] : 0.f;
        for (int j = 0; j < taps; ++j) {
            float hv[VEC], wv[VEC];
            if (j == back) {
#pragma unroll
                for (int v = 0; v < VEC; ++v) hv[v] = x[v];
            } else {
                conv_load<TI, VEC>(h + (size_t)(t - back + j) * ldh + c, hv);
            }
            conv_load<float, VEC>(w + (size_t)j * C + c, wv);
#pragma unroll
            for (int v = 0; v < VEC; ++v) a0[v] = fmaf(wv[v], hv[v], a0[v]);
            if (n_filters > 1) {
                conv_load<float, VEC>(w1 + (size_t)j * C + c, wv);
#pragma unroll
                for (int v = 0; v < VEC; ++v) a1[v] = fmaf(wv[v], hv[v], a1[v]);
            }
        }
#pragma unroll
        for (int v = 0; v < VEC; ++v) a0[v] = conv_finish(a0[v], bias, c + v, act);
        conv_store<TO, VEC>(out0 + (size_t)t * C + c, a0);
        if (n_filters > 1) {
#pragma unroll
            for (int v = 0; v < VEC; ++v) a1[v] = conv_finish(a1[v], bias ? bias + C : nullptr, c + v, act);
            conv_store<TO, VEC>(out1 + (size_t)t * C + c, a1);
        }
        return;
    }
    if (i != 0) return;
    for (int v = 0; v < VEC; ++v)
        conv_entry_head<TI, TO>(h, ldh, bias, act, w, state, out0, out1, q_start, start_pos, slot_ids, e, first, c + v, C, taps, n_filters,
                                residual, state_stride);
}

}  // namespace

// h [n_tokens, C] in `in_dtype` with `ldh` elements from row to row; bias float32 [n_filters, C] or null; act 0: none,
// 1: silu; w float32 [n_filters, taps, C]; state float32 [slots, taps - 1, C] with `state_stride`
// floats from slot to slot (at least (taps - 1) * C; may be null when taps == 1); out0, out1 (out1 only with two filters) and copy (may be null) [n_tokens, C] in `out_dtype`.
extern "C" int qi_short_conv(const void* h, int in_dtype, long long ldh, const float* bias, int act, const float* w, float* state,
                             void* out0, void* out1, void* copy,
                             int out_dtype, const int* token_req, const int* q_start, const int* start_pos,
                             const int* slot_ids, int n_tokens, int channels, int taps, int n_filters, int residual,
                             long long state_stride, cudaStream_t stream) {
    QI_REQUIRE(taps == 1 || state_stride >= (long long)(taps - 1) * channels, "short_conv: the slots of the state overlap");
    QI_REQUIRE(n_tokens >= 0 && channels > 0 && ldh >= channels, "short_conv: bad sizes n=%d channels=%d", n_tokens, channels);
    QI_REQUIRE(taps >= 1 && taps <= kMaxTaps, "short_conv: %d taps are outside 1..%d", taps, kMaxTaps);
    QI_REQUIRE(n_filters == 1 || n_filters == 2, "short_conv: one or two filters a launch, got %d", n_filters);
    QI_REQUIRE(taps == 1 || state, "short_conv: a filter of more than one tap needs its state");
    QI_REQUIRE(out0 && (n_filters == 1 || out1), "short_conv: an output is missing");
    QI_REQUIRE(act == 0 || act == 1, "short_conv: unknown activation code %d", act);
    if (n_tokens == 0) return 0;
    // four channels a thread where every row of every operand starts on a 16-byte boundary (8 for bfloat16) and the step
    // has rows enough to fill the device so; a step of few rows (single tokens, each the first of its entry, whose thread
    // walks the old state) keeps a thread a channel. Both forms add in the same order: a row's result is the same.
    auto aligned = [](const void* p, size_t bytes) { return p == nullptr || reinterpret_cast<size_t>(p) % bytes == 0; };
    const size_t in_bytes = (in_dtype == qi::kF32 ? 4 : 2) * 4, out_bytes = (out_dtype == qi::kF32 ? 4 : 2) * 4;
    const bool wide = n_tokens >= 256 && channels % 4 == 0 && ldh % 4 == 0 && aligned(h, in_bytes) && aligned(w, 16) && aligned(out0, out_bytes) &&
                      aligned(out1, out_bytes) && aligned(copy, out_bytes);
    const size_t total = (size_t)n_tokens * (wide ? channels / 4 : channels);
    QI_REQUIRE((total + 255) / 256 <= 0x7fffffffull, "short_conv: grid too large");
#define QI_CONV(VEC)                                                                                                                  \
    qi::launch(short_conv_kernel<TI, TO, VEC>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, (const TI*)h, ldh, bias, act, \
               w, state, (TO*)out0, (TO*)out1, (TO*)copy, token_req, q_start, start_pos, slot_ids, n_tokens, channels, taps, n_filters,   \
               residual, state_stride)
    QI_DISPATCH_DTYPE(in_dtype, TI, {
        QI_DISPATCH_DTYPE(out_dtype, TO, {
            if (wide) QI_CONV(4); else QI_CONV(1);
        });
    });
#undef QI_CONV
    return qi::check_launch("short_conv");
}

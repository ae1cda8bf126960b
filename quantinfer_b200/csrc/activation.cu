// The gate of a gated feed-forward: out[t, i] = act(gate[t, i]) * up[t, i], where one fused
// projection wrote gate and up into one row of width 2I: either side by side
// (gate_up[t, 0:I] and gate_up[t, I:2I]) or interleaved (gate_up[t, 2i] and
// gate_up[t, 2i + 1]; the layout whose pairs one GEMM epilogue thread holds).
// The activation is a parameter of the feed-forward part:
//   silu       g / (1 + exp(-g)), in the reference's form (division, then the product;
//              backends/cpu/src/backend.rs:224-238, :235): the only one the reference's model uses
//   gelu       g * 0.5 * (1 + erf(g / sqrt 2))
//   gelu_tanh  g * 0.5 * (1 + tanh(sqrt(2 / pi) * (g + 0.044715 g^3)))
//   relu       max(g, 0)
//   relu2      max(g, 0)^2
//   tanh       tanh(g)
// (the reference's description of a model names Gelu and Relu beside Silu and uses neither,
// crates/quantinfer-model/src/semantic.rs:26-30). All in 32-bit.
#include "common.cuh"

namespace {

enum Act : int { kSilu = 0, kGelu = 1, kGeluTanh = 2, kRelu = 3, kRelu2 = 4, kTanh = 5 };

template <int ACT> __device__ __forceinline__ float act(float g) {
    if (ACT == kSilu) return g / (1.0f + expf(-g));
    if (ACT == kGelu) return g * 0.5f * (1.0f + erff(g * 0.70710678118654752f));
    if (ACT == kGeluTanh) return g * 0.5f * (1.0f + tanhf(0.79788456080286536f * (g + 0.044715f * g * g * g)));
    if (ACT == kRelu2) { const float r = fmaxf(g, 0.f); return r * r; }
    if (ACT == kTanh) return tanhf(g);
    return fmaxf(g, 0.f);
}

template <typename T, int ACT>
__global__ void act_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int n_tokens,
                               int inter, int interleaved) {
    qi::pdl_enter();
    const size_t total = (size_t)n_tokens * inter;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / inter, i = idx % inter;
        const T* row = gate_up + t * 2 * inter;
        const float g = qi::to_f32<T>(interleaved ? row[2 * i] : row[i]);
        const float u = qi::to_f32<T>(interleaved ? row[2 * i + 1] : row[inter + i]);
        out[idx] = qi::from_f32<T>(act<ACT>(g) * u);
    }
}

}  // namespace

// activation: 0 silu, 1 gelu (erf), 2 gelu_tanh, 3 relu, 4 relu squared, 5 tanh.
extern "C" int qi_act_mul(const void* gate_up, void* out, int dtype, int n_tokens, int inter, int interleaved,
                          int activation, cudaStream_t stream) {
    QI_REQUIRE(n_tokens >= 0 && inter > 0, "act_mul: bad sizes n=%d inter=%d", n_tokens, inter);
    QI_REQUIRE(activation >= 0 && activation <= 5, "act_mul: unknown activation code %d", activation);
    if (n_tokens == 0) return 0;
    const size_t total = (size_t)n_tokens * inter;
    size_t blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    QI_DISPATCH_DTYPE(dtype, T, {
        const T* in = (const T*)gate_up;
        T* o = (T*)out;
        const dim3 grid((unsigned)blocks), block(256);
        switch (activation) {
            case kSilu: qi::launch(act_mul_kernel<T, kSilu>, grid, block, 0, stream, in, o, n_tokens, inter, interleaved); break;
            case kGelu: qi::launch(act_mul_kernel<T, kGelu>, grid, block, 0, stream, in, o, n_tokens, inter, interleaved); break;
            case kGeluTanh: qi::launch(act_mul_kernel<T, kGeluTanh>, grid, block, 0, stream, in, o, n_tokens, inter, interleaved); break;
            case kRelu2: qi::launch(act_mul_kernel<T, kRelu2>, grid, block, 0, stream, in, o, n_tokens, inter, interleaved); break;
            case kTanh: qi::launch(act_mul_kernel<T, kTanh>, grid, block, 0, stream, in, o, n_tokens, inter, interleaved); break;
            default: qi::launch(act_mul_kernel<T, kRelu>, grid, block, 0, stream, in, o, n_tokens, inter, interleaved); break;
        }
    });
    return qi::check_launch("act_mul");
}

extern "C" int qi_silu_mul(const void* gate_up, void* out, int dtype, int n_tokens, int inter,
                           int interleaved, cudaStream_t stream) {
    return qi_act_mul(gate_up, out, dtype, n_tokens, inter, interleaved, 0, stream);
}

// ---- an activation alone, a sum of gated sublayer outputs, and the soft cap of logits ------------

namespace {

template <typename T, int ACT>
__global__ void activation_kernel(const T* __restrict__ in, T* __restrict__ out, size_t total) {
    qi::pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x)
        out[idx] = qi::from_f32<T>(act<ACT>(qi::to_f32<T>(in[idx])));
}

// out[t, c] = sigmoid(g[t, c] + b0[c]) * y0[t, c] (+ sigmoid(g[t, C + c] + b1[c]) * y1[t, c]), 32-bit out.
template <typename TG, typename TY>
__global__ void gated_sum_kernel(const TG* __restrict__ gates, int ldg, const float* __restrict__ b0,
                                 const float* __restrict__ b1, const TY* __restrict__ y0, const TY* __restrict__ y1,
                                 float* __restrict__ out, int n_tokens, int C) {
    qi::pdl_wait();
    const size_t total = (size_t)n_tokens * C;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / C, c = idx % C;
        const TG* g = gates + t * ldg;
        float v = qi::to_f32<TY>(y0[idx]) / (1.0f + expf(-(qi::to_f32<TG>(g[c]) + b0[c])));
        if (y1) v += qi::to_f32<TY>(y1[idx]) / (1.0f + expf(-(qi::to_f32<TG>(g[C + c]) + b1[c])));
        out[idx] = v;
    }
}

// x[t, c] *= sigmoid(gate[t, c]) in place; the gate's rows lie `ldg` elements apart.
template <typename T, typename TG>
__global__ void sigmoid_gate_kernel(T* __restrict__ x, const TG* __restrict__ gate, long long ldg, int n_tokens, int C) {
    qi::pdl_wait();
    const size_t total = (size_t)n_tokens * C;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / C, c = idx % C;
        x[idx] = qi::from_f32<T>(qi::to_f32<T>(x[idx]) / (1.0f + expf(-qi::to_f32<TG>(gate[t * ldg + c]))));
    }
}

__global__ void softcap_kernel(float* __restrict__ x, size_t total, float cap, float inv_cap) {
    qi::pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x)
        x[idx] = cap * tanhf(x[idx] * inv_cap);
}

unsigned blocks_for(size_t total) {
    size_t blocks = (total + 255) / 256;
    return (unsigned)(blocks > 148 * 32 ? 148 * 32 : blocks);
}

}  // namespace

// out = act(in), elementwise, both [n] in `dtype`; 32-bit arithmetic.
extern "C" int qi_activation(const void* in, void* out, int dtype, long long n, int activation, cudaStream_t stream) {
    QI_REQUIRE(n >= 0, "activation: bad size");
    QI_REQUIRE(activation >= 0 && activation <= 5, "activation: unknown activation code %d", activation);
    if (n == 0) return 0;
    const dim3 grid(blocks_for((size_t)n)), block(256);
    QI_DISPATCH_DTYPE(dtype, T, {
        switch (activation) {
            case kSilu: qi::launch(activation_kernel<T, kSilu>, grid, block, 0, stream, (const T*)in, (T*)out, (size_t)n); break;
            case kGelu: qi::launch(activation_kernel<T, kGelu>, grid, block, 0, stream, (const T*)in, (T*)out, (size_t)n); break;
            case kGeluTanh: qi::launch(activation_kernel<T, kGeluTanh>, grid, block, 0, stream, (const T*)in, (T*)out, (size_t)n); break;
            case kRelu2: qi::launch(activation_kernel<T, kRelu2>, grid, block, 0, stream, (const T*)in, (T*)out, (size_t)n); break;
            case kTanh: qi::launch(activation_kernel<T, kTanh>, grid, block, 0, stream, (const T*)in, (T*)out, (size_t)n); break;
            default: qi::launch(activation_kernel<T, kRelu>, grid, block, 0, stream, (const T*)in, (T*)out, (size_t)n); break;
        }
    });
    return qi::check_launch("activation");
}

// The sum of one or two sublayer outputs, each scaled by a sigmoid gate: gates [n, ldg] holds the gates'
// pre-activations (the first C columns for y0, the next C for y1), b0 and b1 their biases (float32 [C]);
// y1 and b1 may be null (one sublayer). out float32 [n, C].
extern "C" int qi_gated_sum(const void* gates, int gates_dtype, int ldg, const float* b0, const float* b1,
                            const void* y0, const void* y1, int y_dtype, float* out, int n_tokens, int channels,
                            cudaStream_t stream) {
    QI_REQUIRE(n_tokens >= 0 && channels > 0, "gated_sum: bad sizes n=%d channels=%d", n_tokens, channels);
    QI_REQUIRE(ldg >= (y1 ? 2 : 1) * channels, "gated_sum: the gates' rows are too short");
    QI_REQUIRE(gates && b0 && y0 && out && (!y1 || b1), "gated_sum: an argument is missing");
    if (n_tokens == 0) return 0;
    const dim3 grid(blocks_for((size_t)n_tokens * channels)), block(256);
    QI_DISPATCH_DTYPE(gates_dtype, TG, {
        QI_DISPATCH_DTYPE(y_dtype, TY, {
            qi::launch(gated_sum_kernel<TG, TY>, grid, block, 0, stream, (const TG*)gates, ldg, b0, b1, (const TY*)y0, (const TY*)y1,
                       out, n_tokens, channels);
        });
    });
    return qi::check_launch("gated_sum");
}

// x = cap * tanh(x / cap) in place, float32 [n].
// x [n, C] in `dtype`, multiplied in place by sigmoid(gate), gate [n, >= C] in `gate_dtype` with rows `ldg` elements apart.
extern "C" int qi_sigmoid_gate(void* x, int dtype, const void* gate, int gate_dtype, long long ldg, int n_tokens, int C,
                               cudaStream_t stream) {
    QI_REQUIRE(n_tokens >= 0 && C > 0 && ldg >= C, "sigmoid_gate: bad sizes");
    if (n_tokens == 0) return 0;
    const size_t total = (size_t)n_tokens * C;
    QI_DISPATCH_DTYPE(dtype, T, {
        QI_DISPATCH_DTYPE(gate_dtype, TG, {
            qi::launch(sigmoid_gate_kernel<T, TG>, dim3(blocks_for(total)), dim3(256), 0, stream, (T*)x, (const TG*)gate, ldg, n_tokens, C);
        });
    });
    return qi::check_launch("sigmoid_gate");
}

extern "C" int qi_softcap(float* x, long long n, float cap, cudaStream_t stream) {
    QI_REQUIRE(n >= 0 && cap > 0.f, "softcap: bad size or cap");
    if (n == 0) return 0;
    qi::launch(softcap_kernel, dim3(blocks_for((size_t)n)), dim3(256), 0, stream, x, (size_t)n, cap, 1.0f / cap);
    return qi::check_launch("softcap");
}

// ---- the clamped gated unit of small expert feed-forwards ------------------------------------------------
//   g = min(gate, limit) ; u = clamp(up, -limit, limit) ; out = g * sigmoid(alpha * g) * (u + 1)
// gate and up side by side or interleaved in rows of 2 I, as for act_mul; 32-bit arithmetic.
namespace {

template <typename T>
__global__ void glu_clamped_kernel(const T* __restrict__ gate_up, T* __restrict__ out, size_t n_rows, int inter, int interleaved,
                                   float limit, float alpha) {
    qi::pdl_wait();
    const size_t total = n_rows * inter;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / inter, i = idx % inter;
        const T* row = gate_up + t * 2 * inter;
        const float g = fminf(qi::to_f32<T>(interleaved ? row[2 * i] : row[i]), limit);
        const float u = fminf(fmaxf(qi::to_f32<T>(interleaved ? row[2 * i + 1] : row[inter + i]), -limit), limit);
        out[idx] = qi::from_f32<T>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
    }
}

}  // namespace

extern "C" int qi_glu_clamped(const void* gate_up, void* out, int dtype, long long n_rows, int inter, int interleaved, float limit,
                              float alpha, cudaStream_t stream) {
    QI_REQUIRE(n_rows >= 0 && inter > 0, "glu_clamped: bad sizes");
    if (n_rows == 0) return 0;
    QI_DISPATCH_DTYPE(dtype, T, {
        qi::launch(glu_clamped_kernel<T>, dim3(blocks_for((size_t)n_rows * inter)), dim3(256), 0, stream, (const T*)gate_up, (T*)out,
                   (size_t)n_rows, inter, interleaved, limit, alpha);
    });
    return qi::check_launch("glu_clamped");
}

// A selective state-space recurrence with one decay a head (the "state-space duality" form), and the
// gated norm that follows it.
//
// Per head h of P channels with a state S of N x P numbers (32-bit, a request's state of fixed size):
//
//     dt_t = softplus(raw_t + dt_bias_h)                      a_t = exp(-exp(A_log_h) * dt_t)
//     S_t  = a_t * S_(t-1) + dt_t * B_t x_t^T                 y_t = S_t^T C_t + D_h * x_t
//
// B_t and C_t (N numbers each) belong to the head's group (head / (heads / groups)); x, B and C are the
// outputs of the input convolution, raw_t a column of the input projection. Decays, step sizes, the state
// and all sums are 32-bit; x, B, C and raw may be bfloat16.
//
// ssm_scan: one warp walks the tokens of one step entry for `kCols` channels of one head: lane l keeps
// S[n, p] for n = l, l + 32, ... in registers, so a token costs each lane a few multiply-adds and one
// warp sum per channel. The four warps of a block share a head: B, C, x, the step sizes and decays of
// sixteen tokens at a time are brought into shared memory together (one round of loads for sixteen
// steps of the recurrence), and the results leave in rows.
// The state is read once at the entry's first token (zeros at position 0, whatever the slot holds) and
// written once after its last, so one launch serves prompts, portions and single decode tokens alike.
// State layout per slot: [heads, P, N] (N fastest, so a warp's loads are contiguous).
//
// gated_group_rmsnorm: v = y * silu(z); every `width / groups` coordinates are divided by their own root
// mean square (eps inside the root) and multiplied by a gain; 32-bit throughout, output in the activation type.
#include "common.cuh"

namespace {

constexpr int kCols = 8;       // channels a warp
constexpr int kWarps = 4;      // warps a block
constexpr int kBatch = 16;     // tokens whose operands are staged in shared memory at a time

__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

template <typename T, int R>
__global__ void __launch_bounds__(kWarps * 32)
ssm_scan_kernel(const T* __restrict__ xbc, long long ldx, const T* __restrict__ raw_dt, long long lddt,
                const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ d_skip,
                float* __restrict__ state, long long state_stride, float* __restrict__ y,
                const int* __restrict__ q_start, const int* __restrict__ start_pos, const int* __restrict__ slot_ids,
                int heads, int groups, int P, int N, int write_state) {
    // a batch of kBatch tokens' operands, 32-bit: B and C [kBatch][N], x and the results [kBatch][block's columns], dt, decay
    extern __shared__ float sm[];
    constexpr int kBlockCols = kWarps * kCols;
    float* Bs = sm;
    float* Cs = Bs + kBatch * N;
    float* xs = Cs + kBatch * N;
    float* ys = xs + kBatch * kBlockCols;
    float* dts = ys + kBatch * kBlockCols;
    float* decs = dts + kBatch;
    qi::pdl_wait();
    const int h = blockIdx.x, e = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pb = blockIdx.z * kBlockCols;          // the block's first channel of the head
    const int p0 = pb + warp * kCols;                // the warp's
    const int g = h / (heads / groups);
    const int inner = heads * P;
    const int t0 = q_start[e], t1 = q_start[e + 1];
    const float A = -expf(a_log[h]), bias = dt_bias[h], D = d_skip[h];
    float* st = state + (size_t)slot_ids[e] * state_stride + ((size_t)h * P + p0) * N;

    float S[kCols][R];
    const bool fresh = start_pos[e] == 0;
#pragma unroll
    for (int c = 0; c < kCols; ++c)
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int n = lane + 32 * r;
            S[c][r] = (!fresh && n < N && p0 + c < P) ? st[(size_t)c * N + n] : 0.f;
        }

    const size_t xoff = (size_t)h * P + pb, boff = (size_t)inner + (size_t)g * N, coff = (size_t)inner + (size_t)groups * N + (size_t)g * N;
    for (int tb = t0; tb < t1; tb += kBatch) {
        const int nb = min(kBatch, t1 - tb);
        __syncthreads();                              // the batch before is consumed and written
        for (int i = warp; i < nb; i += kWarps) {     // a warp brings whole rows: no division in the loop
            const T* rb = xbc + (size_t)(tb + i) * ldx + boff;
            const T* rc = xbc + (size_t)(tb + i) * ldx + coff;
            for (int n = lane; n < N; n += 32) {
                Bs[i * N + n] = qi::to_f32<T>(rb[n]);
                Cs[i * N + n] = qi::to_f32<T>(rc[n]);
            }
        }
        for (int idx = threadIdx.x; idx < nb * kBlockCols; idx += blockDim.x) {
            const int i = idx / kBlockCols, c = idx % kBlockCols;
            xs[idx] = pb + c < P ? qi::to_f32<T>(xbc[(size_t)(tb + i) * ldx + xoff + c]) : 0.f;
        }
        if ((int)threadIdx.x < nb) {
            const float dt = softplus_f(qi::to_f32<T>(raw_dt[(size_t)(tb + threadIdx.x) * lddt + h]) + bias);
            dts[threadIdx.x] = dt;
            decs[threadIdx.x] = expf(A * dt);
        }
        __syncthreads();
        for (int i = 0; i < nb; ++i) {
            const float dt = dts[i], a = decs[i];
            float B[R], C[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int n = lane + 32 * r;
                B[r] = n < N ? Bs[i * N + n] : 0.f;
                C[r] = n < N ? Cs[i * N + n] : 0.f;
            }
            float part[kCols];
#pragma unroll
            for (int c = 0; c < kCols; ++c) {
                const float dx = dt * xs[i * kBlockCols + warp * kCols + c];
                part[c] = 0.f;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    S[c][r] = fmaf(a, S[c][r], dx * B[r]);
                    part[c] = fmaf(S[c][r], C[r], part[c]);
                }
            }
            if (!y) continue;          // a pass that is after the end state only
            // four channels' sums over the warp in six exchanges: halves trade channels, then quarters, then the
            // eight lanes that are left add up; lanes 0, 8, 16 and 24 end up with channels 0, 1, 2 and 3 of the four
            static_assert(kCols % 4 == 0, "the exchange below takes four channels at a time");
            const bool up16 = lane & 16, up8 = lane & 8;
#pragma unroll
            for (int q4 = 0; q4 < kCols; q4 += 4) {
                float k0 = up16 ? part[q4 + 2] : part[q4], k1 = up16 ? part[q4 + 3] : part[q4 + 1];
                k0 += __shfl_xor_sync(0xffffffffu, up16 ? part[q4] : part[q4 + 2], 16);
                k1 += __shfl_xor_sync(0xffffffffu, up16 ? part[q4 + 1] : part[q4 + 3], 16);
                float k = up8 ? k1 : k0;
                k += __shfl_xor_sync(0xffffffffu, up8 ? k0 : k1, 8);
                k += __shfl_xor_sync(0xffffffffu, k, 4);
                k += __shfl_xor_sync(0xffffffffu, k, 2);
                k += __shfl_xor_sync(0xffffffffu, k, 1);
                if ((lane & 7) == 0) {
                    const int c = warp * kCols + q4 + (lane >> 3);
                    ys[i * kBlockCols + c] = k + D * xs[i * kBlockCols + c];
                }
            }
        }
        if (!y) continue;
        __syncthreads();
        for (int idx = threadIdx.x; idx < nb * kBlockCols; idx += blockDim.x) {
            const int i = idx / kBlockCols, c = idx % kBlockCols;
            if (pb + c < P) y[(size_t)(tb + i) * inner + xoff + c] = ys[idx];
        }
    }
    if (!write_state) return;
#pragma unroll
    for (int c = 0; c < kCols; ++c)
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int n = lane + 32 * r;
            if (n < N && p0 + c < P) st[(size_t)c * N + n] = S[c][r];
        }
}

// The same recurrence with a thread (or two neighbours) a channel: the thread keeps its channel's column S[0 .. N) in
// registers (two threads: alternate groups of four rows each), so a token's output is a sum inside one thread (two: one
// exchange) and B_t, C_t come as broadcast 16-byte loads from shared memory. For entries of many tokens (the second pass over segments) and states of at most 128 rows; a
// single decode token is better off with ssm_scan_kernel, whose warps read a slot's state in contiguous rows.
constexpr int kColChannels = 64;      // channels of a head a block takes

// kEndOnly: no outputs, the end state alone by the unrolled sum that ssm_end_state_kernel describes (y is not touched,
// C is not read, the state is always written).
template <typename T, int NP, int SPLIT, bool kEndOnly>
__global__ void __launch_bounds__(kColChannels * SPLIT)
ssm_scan_cols_kernel(const T* __restrict__ xbc, long long ldx, const T* __restrict__ raw_dt, long long lddt,
                     const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ d_skip,
                     float* __restrict__ state, long long state_stride, float* __restrict__ y,
                     const int* __restrict__ q_start, const int* __restrict__ start_pos, const int* __restrict__ slot_ids,
                     int heads, int groups, int P, int N, int write_state, int vec_ok) {
    __shared__ __align__(16) float Bs[kBatch * NP];
    __shared__ __align__(16) float Cs[kBatch * NP];
    __shared__ float xs[kBatch * kColChannels];
    __shared__ float dts[kBatch], decs[kBatch + 1];      // kEndOnly: decs holds the tokens' weights and the batch's decay
    qi::pdl_wait();
    const int h = blockIdx.x, e = blockIdx.y;
    constexpr int kColThreads = kColChannels * SPLIT, NT = NP / SPLIT;     // NT: rows of the state a thread keeps
    const int half = (int)threadIdx.x % SPLIT;
    const int pb = blockIdx.z * kColChannels, p = pb + (int)threadIdx.x / SPLIT;
    const bool valid = p < P;
    auto row_of = [&](int k) { return ((k >> 2) * SPLIT + half) * 4 + (k & 3); };      // the k-th row this thread keeps
    const int g = h / (heads / groups);
    const int inner = heads * P;
    const int t0 = q_start[e], t1 = q_start[e + 1];
    const float A = -expf(a_log[h]), bias = dt_bias[h], D = d_skip[h];
    float* st = state + (size_t)slot_ids[e] * state_stride + ((size_t)h * P + (valid ? p : 0)) * N;
    float S[NT];
    const bool load = valid && start_pos[e] != 0;
#pragma unroll
    for (int k = 0; k < NT; ++k) S[k] = (load && row_of(k) < N) ? st[row_of(k)] : 0.f;
    const size_t xcol = (size_t)h * P + (valid ? p : 0), boff = (size_t)inner + (size_t)g * N, coff = boff + (size_t)groups * N;

    // bfloat16 rows that allow 16-byte loads: the next batch's B and C are requested (eight numbers a load, all of a
    // thread's loads in flight together) before this batch's arithmetic and put into shared memory after it
    constexpr bool kHalf = sizeof(T) == 2;
    constexpr int kPf = (kEndOnly ? 2 : 4) * NP / kColThreads;     // 1 or 2 matrices x kBatch rows x NP / 8 vectors over the block's threads
    const bool vec = kHalf && vec_ok;
    uint4 pf[kPf];
    float pf_dt = 0.f;
    T pf_x[kBatch / SPLIT];                            // the thread's channel at every SPLIT-th token of the next batch
    auto fetch = [&](int tb, int nb) {
#pragma unroll
        for (int k = 0; k < kPf; ++k) {
            const int v = (int)threadIdx.x + kColThreads * k;
            const int m = v / (kBatch * (NP / 8)), rem = v % (kBatch * (NP / 8)), i = rem / (NP / 8), n = (rem % (NP / 8)) * 8;
            pf[k] = (i < nb && n < N) ? *reinterpret_cast<const uint4*>(xbc + (size_t)(tb + i) * ldx + (m ? coff : boff) + n)
                                      : make_uint4(0u, 0u, 0u, 0u);
        }
    };
    auto fetch_dt = [&](int tb, int nb) {
        if ((int)threadIdx.x < nb) pf_dt = qi::to_f32<T>(raw_dt[(size_t)(tb + threadIdx.x) * lddt + h]);
#pragma unroll
        for (int k = 0; k < kBatch / SPLIT; ++k) {
            const int i = k * SPLIT + half;
            pf_x[k] = (valid && i < nb) ? xbc[(size_t)(tb + i) * ldx + xcol] : qi::from_f32<T>(0.f);
        }
    };
    if (t0 < t1) {
        if (vec) fetch(t0, min(kBatch, t1 - t0));
        fetch_dt(t0, min(kBatch, t1 - t0));
    }
    for (int tb = t0; tb < t1; tb += kBatch) {
        const int nb = min(kBatch, t1 - tb);
        __syncthreads();                               // the batch before has been read
        if (vec) {
#pragma unroll
            for (int k = 0; k < kPf; ++k) {
                const int v = (int)threadIdx.x + kColThreads * k;
                const int m = v / (kBatch * (NP / 8)), rem = v % (kBatch * (NP / 8));
                float* dst = (m ? Cs : Bs) + rem * 8;
                const uint32_t w[4] = {pf[k].x, pf[k].y, pf[k].z, pf[k].w};
                *reinterpret_cast<float4*>(dst) = make_float4(__uint_as_float(w[0] << 16), __uint_as_float(w[0] & 0xffff0000u),
                                                              __uint_as_float(w[1] << 16), __uint_as_float(w[1] & 0xffff0000u));
                *reinterpret_cast<float4*>(dst + 4) = make_float4(__uint_as_float(w[2] << 16), __uint_as_float(w[2] & 0xffff0000u),
                                                                  __uint_as_float(w[3] << 16), __uint_as_float(w[3] & 0xffff0000u));
            }
        } else {
            for (int idx = threadIdx.x; idx < nb * NP; idx += kColThreads) {     // rows beyond N are zeros: those S stay zero
                const int i = idx / NP, n = idx % NP;
                const T* row = xbc + (size_t)(tb + i) * ldx;
                Bs[idx] = n < N ? qi::to_f32<T>(row[boff + n]) : 0.f;
                if (!kEndOnly) Cs[idx] = n < N ? qi::to_f32<T>(row[coff + n]) : 0.f;
            }
        }
        if (!kEndOnly) {
            if ((int)threadIdx.x < nb) {
                const float dt = softplus_f(pf_dt + bias);
                dts[threadIdx.x] = dt;
                decs[threadIdx.x] = expf(A * dt);
            }
        } else if (threadIdx.x < 32) {       // lane i: the step sizes from token i on, added up over the lanes behind it
            static_assert(kBatch <= 16, "the sums below cover sixteen lanes");
            const float dt = (int)threadIdx.x < nb ? softplus_f(pf_dt + bias) : 0.f;
            float from = dt;
#pragma unroll
            for (int d = 1; d < kBatch; d *= 2) {
                const float v = __shfl_down_sync(0xffffffffu, from, d);
                if ((int)threadIdx.x + d < kBatch) from += v;
            }
            if ((int)threadIdx.x < nb) decs[threadIdx.x] = dt * expf(A * (from - dt));
            if (threadIdx.x == 0) decs[kBatch] = expf(A * from);
        }
#pragma unroll
        for (int k = 0; k < kBatch / SPLIT; ++k) xs[(k * SPLIT + half) * kColChannels + (int)threadIdx.x / SPLIT] = qi::to_f32<T>(pf_x[k]);
        __syncthreads();
        if (tb + kBatch < t1) {
            if (vec) fetch(tb + kBatch, min(kBatch, t1 - tb - kBatch));
            fetch_dt(tb + kBatch, min(kBatch, t1 - tb - kBatch));
        }
        if (kEndOnly) {
            const float whole = decs[kBatch];
#pragma unroll
            for (int k = 0; k < NT; ++k) S[k] *= whole;
            for (int i = 0; i < nb; ++i) {
                const float wx = decs[i] * xs[i * kColChannels + (int)threadIdx.x / SPLIT];
                const float4* b4 = reinterpret_cast<const float4*>(Bs + i * NP);
#pragma unroll
                for (int n = 0; n < NT; n += 4) {
                    const float4 b = b4[(n >> 2) * SPLIT + half];
                    S[n] = fmaf(wx, b.x, S[n]);
                    S[n + 1] = fmaf(wx, b.y, S[n + 1]);
                    S[n + 2] = fmaf(wx, b.z, S[n + 2]);
                    S[n + 3] = fmaf(wx, b.w, S[n + 3]);
                }
            }
            continue;
        }
        for (int i = 0; i < nb; ++i) {
            const float a = decs[i], x = xs[i * kColChannels + (int)threadIdx.x / SPLIT], dx = dts[i] * x;
            const float4* b4 = reinterpret_cast<const float4*>(Bs + i * NP);
            const float4* c4 = reinterpret_cast<const float4*>(Cs + i * NP);
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int n = 0; n < NT; n += 4) {
                const float4 b = b4[(n >> 2) * SPLIT + half], c = c4[(n >> 2) * SPLIT + half];
                S[n] = fmaf(a, S[n], dx * b.x);
                S[n + 1] = fmaf(a, S[n + 1], dx * b.y);
                S[n + 2] = fmaf(a, S[n + 2], dx * b.z);
                S[n + 3] = fmaf(a, S[n + 3], dx * b.w);
                acc[0] = fmaf(S[n], c.x, acc[0]);
                acc[1] = fmaf(S[n + 1], c.y, acc[1]);
                acc[2] = fmaf(S[n + 2], c.z, acc[2]);
                acc[3] = fmaf(S[n + 3], c.w, acc[3]);
            }
            float sum = (acc[0] + acc[1]) + (acc[2] + acc[3]);
            if (SPLIT == 2) sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            if (valid && half == 0) y[(size_t)(tb + i) * inner + xcol] = sum + D * x;
        }
    }
    if (!(write_state || kEndOnly) || !valid) return;
#pragma unroll
    for (int k = 0; k < NT; ++k)
        if (row_of(k) < N) st[row_of(k)] = S[k];
}

// The end state alone (no outputs), for the first pass over segments: within a batch of kBatch tokens the recurrence is
// unrolled, S_end = exp(A sum_u dt_u) S_begin + sum_s exp(A sum_(u > s) dt_u) dt_s B_s x_s^T, so a state element costs one
// multiply-add a token (the weight times x is formed once a token and channel) and one multiply a batch, instead of a
// multiply and a multiply-add a token; C is not read. Step sizes, their sums, the decays and all sums are 32-bit.
template <typename T, int R>
__global__ void __launch_bounds__(kWarps * 32)
ssm_end_state_kernel(const T* __restrict__ xbc, long long ldx, const T* __restrict__ raw_dt, long long lddt,
                     const float* __restrict__ dt_bias, const float* __restrict__ a_log, float* __restrict__ state,
                     long long state_stride, const int* __restrict__ q_start, const int* __restrict__ start_pos,
                     const int* __restrict__ slot_ids, int heads, int groups, int P, int N) {
    extern __shared__ float sm[];
    constexpr int kBlockCols = kWarps * kCols;
    float* Bs = sm;                              // [kBatch][N]
    float* xs = Bs + kBatch * N;                 // [kBatch][block's columns]
    float* dts = xs + kBatch * kBlockCols;       // [kBatch] step sizes
    float* ws = dts + kBatch;                    // [kBatch] a token's weight in the batch's end state, then the batch's decay
    qi::pdl_wait();
    const int h = blockIdx.x, e = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pb = blockIdx.z * kBlockCols, p0 = pb + warp * kCols;
    const int g = h / (heads / groups);
    const int inner = heads * P;
    const int t0 = q_start[e], t1 = q_start[e + 1];
    const float A = -expf(a_log[h]), bias = dt_bias[h];
    float* st = state + (size_t)slot_ids[e] * state_stride + ((size_t)h * P + p0) * N;
    float S[kCols][R];
    const bool fresh = start_pos[e] == 0;
#pragma unroll
    for (int c = 0; c < kCols; ++c)
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int n = lane + 32 * r;
            S[c][r] = (!fresh && n < N && p0 + c < P) ? st[(size_t)c * N + n] : 0.f;
        }
    const size_t xoff = (size_t)h * P + pb, boff = (size_t)inner + (size_t)g * N;
    for (int tb = t0; tb < t1; tb += kBatch) {
        const int nb = min(kBatch, t1 - tb);
        __syncthreads();
        for (int i = warp; i < nb; i += kWarps) {
            const T* rb = xbc + (size_t)(tb + i) * ldx + boff;
            for (int n = lane; n < N; n += 32) Bs[i * N + n] = qi::to_f32<T>(rb[n]);
        }
        for (int idx = threadIdx.x; idx < nb * kBlockCols; idx += blockDim.x) {
            const int i = idx / kBlockCols, c = idx % kBlockCols;
            xs[idx] = pb + c < P ? qi::to_f32<T>(xbc[(size_t)(tb + i) * ldx + xoff + c]) : 0.f;
        }
        if ((int)threadIdx.x < nb) dts[threadIdx.x] = softplus_f(qi::to_f32<T>(raw_dt[(size_t)(tb + threadIdx.x) * lddt + h]) + bias);
        __syncthreads();
        if ((int)threadIdx.x <= nb) {            // thread i: the step sizes after token i; thread nb: the whole batch's
            const int i = (int)threadIdx.x == nb ? -1 : (int)threadIdx.x;
            float after = 0.f;
            for (int u = nb - 1; u > i; --u) after += dts[u];
            ws[threadIdx.x == nb ? kBatch : i] = (i < 0 ? 1.f : dts[i]) * expf(A * after);
        }
        __syncthreads();
        const float whole = ws[kBatch];
#pragma unroll
        for (int c = 0; c < kCols; ++c)
#pragma unroll
            for (int r = 0; r < R; ++r) S[c][r] *= whole;
        for (int i = 0; i < nb; ++i) {
            const float w = ws[i];
            float B[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int n = lane + 32 * r;
                B[r] = n < N ? Bs[i * N + n] : 0.f;
            }
#pragma unroll
            for (int c = 0; c < kCols; ++c) {
                const float wx = w * xs[i * kBlockCols + warp * kCols + c];
#pragma unroll
                for (int r = 0; r < R; ++r) S[c][r] = fmaf(wx, B[r], S[c][r]);
            }
        }
    }
#pragma unroll
    for (int c = 0; c < kCols; ++c)
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int n = lane + 32 * r;
            if (n < N && p0 + c < P) st[(size_t)c * N + n] = S[c][r];
        }
}

// Long entries are cut into segments that run side by side (the recurrence is linear in the state):
//   1. ssm_scan over the segments as if each began a sequence: segment k's own contribution L_k to its end state;
//   2. ssm_chain (this kernel): per entry, in order, in_k = carry ; carry = exp(A * sum of dt over k) * carry + L_k,
//      beginning with the request's state (zeros at position 0) and ending with the request's new state;
//   3. ssm_scan over the segments once more, each from its true state in_k, for the outputs.
// seg_state [segments, heads, P, N] holds L_k on entry and in_k on exit. A block takes 256 numbers of one head's state of one entry.
constexpr int kChainSpan = 256;     // numbers of a head's state a block of the chain takes

template <typename T>
__global__ void __launch_bounds__(256)
ssm_chain_kernel(float* __restrict__ seg_state, float* __restrict__ state, long long state_stride,
                 const T* __restrict__ raw_dt, long long lddt, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                 const int* __restrict__ seg_q_start, const int* __restrict__ entry_seg, const int* __restrict__ start_pos,
                 const int* __restrict__ slot_ids, int heads, int P, int N) {
    extern __shared__ float decay[];          // one a segment of this entry
    qi::pdl_wait();
    const int h = blockIdx.x, e = blockIdx.y;
    const int s0 = entry_seg[e], s1 = entry_seg[e + 1];
    const float A = -expf(a_log[h]), bias = dt_bias[h];
    // eight threads a segment add up its step sizes
    for (int k0 = s0; k0 < s1; k0 += blockDim.x / 8) {
        const int k = k0 + (int)threadIdx.x / 8, part = threadIdx.x & 7;
        float sum = 0.f;
        if (k < s1)
            for (int t = seg_q_start[k] + part; t < seg_q_start[k + 1]; t += 8)
                sum += softplus_f(qi::to_f32<T>(raw_dt[(size_t)t * lddt + h]) + bias);
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        sum += __shfl_xor_sync(0xffffffffu, sum, 4);
        if (k < s1 && part == 0) decay[k - s0] = expf(A * sum);
    }
    __syncthreads();
    const size_t per_head = (size_t)P * N, per_seg = (size_t)heads * per_head;
    float* st = state + (size_t)slot_ids[e] * state_stride + (size_t)h * per_head;
    const bool fresh = start_pos[e] == 0;
    const size_t lo = (size_t)blockIdx.z * kChainSpan, hi = lo + kChainSpan < per_head ? lo + kChainSpan : per_head;
    for (size_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        float carry = fresh ? 0.f : st[i];
        float* cell = seg_state + (size_t)s0 * per_seg + (size_t)h * per_head + i;
        for (int k = s0; k < s1; k += 8) {          // eight segments' loads in flight at a time
            float local[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) local[j] = k + j < s1 ? cell[(size_t)j * per_seg] : 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (k + j < s1) {
                    cell[(size_t)j * per_seg] = carry;
                    carry = fmaf(decay[k + j - s0], carry, local[j]);
                }
            }
            cell += 8 * per_seg;
        }
        st[i] = carry;
    }
}

// mode 0: norm(y * silu(z)) * gain (the gate before the norm); mode 1: norm(y) * gain * silu(z); mode 2: norm(y) * gain *
// sigmoid(z); mode 3: norm(y) * gain * z (a gate that carries its activation already); all times out_scale.
template <typename TZ, typename TO>
__global__ void __launch_bounds__(256)
gated_group_rmsnorm_kernel(const float* __restrict__ y, const TZ* __restrict__ z, long long ldz, const float* __restrict__ gain,
                           float eps, TO* __restrict__ out, int width, int groups, int mode, float out_scale) {
    __shared__ float scratch[32];
    qi::pdl_wait();
    const int t = blockIdx.x, grp = blockIdx.y;
    const int gw = width / groups;
    const float* yr = y + (size_t)t * width + (size_t)grp * gw;
    const TZ* zr = z + (size_t)t * ldz + (size_t)grp * gw;
    float ss = 0.f;
    for (int i = threadIdx.x; i < gw; i += blockDim.x) {
        float v = yr[i];
        if (mode == 0) {
            const float zz = qi::to_f32<TZ>(zr[i]);
            v *= zz / (1.0f + expf(-zz));
        }
        ss = fmaf(v, v, ss);
    }
    const float total = qi::block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(total / (float)gw + eps);
    for (int i = threadIdx.x; i < gw; i += blockDim.x) {
        const float zz = qi::to_f32<TZ>(zr[i]);
        const float sg = 1.0f / (1.0f + expf(-zz));
        float v = yr[i];
        if (mode == 0) v *= zz * sg;
        v = v * inv * gain[(size_t)grp * gw + i];
        if (mode == 1) v *= zz * sg;
        else if (mode == 2) v *= sg;
        else if (mode == 3) v *= zz;
        out[(size_t)t * width + (size_t)grp * gw + i] = qi::from_f32<TO>(v * out_scale);
    }
}

// The same for narrow groups (up to kNarrowGroup coordinates): a warp a group, eight groups a block, no barrier.
constexpr int kNarrowGroup = 256;

template <typename TZ, typename TO>
__global__ void __launch_bounds__(256)
gated_narrow_group_rmsnorm_kernel(const float* __restrict__ y, const TZ* __restrict__ z, long long ldz, const float* __restrict__ gain,
                                  float eps, TO* __restrict__ out, long long n_groups, int width, int groups, int mode, float out_scale) {
    qi::pdl_wait();
    const long long g = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (g >= n_groups) return;
    const int lane = threadIdx.x & 31;
    const size_t t = (size_t)(g / groups);
    const int grp = (int)(g % groups);
    const int gw = width / groups;
    const float* yr = y + t * width + (size_t)grp * gw;
    const TZ* zr = z + t * ldz + (size_t)grp * gw;
    constexpr int kOwn = kNarrowGroup / 32;
    float v[kOwn], zz[kOwn];
    float ss = 0.f;
#pragma unroll
    for (int m = 0; m < kOwn; ++m) {
        const int i = lane + 32 * m;
        v[m] = i < gw ? yr[i] : 0.f;
        zz[m] = i < gw ? qi::to_f32<TZ>(zr[i]) : 0.f;
        if (mode == 0) v[m] *= zz[m] / (1.0f + expf(-zz[m]));
        ss = fmaf(v[m], v[m], ss);
    }
    const float inv = 1.0f / sqrtf(qi::warp_sum(ss) / (float)gw + eps);
#pragma unroll
    for (int m = 0; m < kOwn; ++m) {
        const int i = lane + 32 * m;
        if (i < gw) {
            const float sg = 1.0f / (1.0f + expf(-zz[m]));
            float r = v[m] * inv * gain[(size_t)grp * gw + i];
            if (mode == 1) r *= zz[m] * sg;
            else if (mode == 2) r *= sg;
            else if (mode == 3) r *= zz[m];
            out[t * width + (size_t)grp * gw + i] = qi::from_f32<TO>(r * out_scale);
        }
    }
}

}  // namespace

// xbc [n, >= heads P + 2 groups N] in `dtype` (x | B | C, `ldx` elements a row); raw_dt [n, >= heads] in `dtype`, column h
// at raw_dt[t * lddt + h]; dt_bias, a_log, d_skip float32 [heads]; state float32, `state_stride` floats from slot to slot,
// [heads, P, N] in a slot; y float32 [n, heads P], or null for a pass that wants the end states only; q_start [entries + 1],
// start_pos, slot_ids [entries]; write_state 0: the end states are not stored.
extern "C" int qi_ssm_scan(const void* xbc, long long ldx, const void* raw_dt, long long lddt, int dtype, const float* dt_bias,
                           const float* a_log, const float* d_skip, float* state, long long state_stride, float* y,
                           const int* q_start, const int* start_pos, const int* slot_ids, int n_entries, int heads,
                           int groups, int P, int N, int write_state, cudaStream_t stream) {
    QI_REQUIRE(n_entries >= 0 && heads > 0 && groups > 0 && P > 0 && N > 0, "ssm_scan: bad sizes");
    QI_REQUIRE(heads % groups == 0, "ssm_scan: %d heads are not a multiple of %d groups", heads, groups);
    QI_REQUIRE(N <= 256, "ssm_scan: a state of %d rows is above this kernel's 256", N);
    QI_REQUIRE(ldx >= (long long)heads * P + 2ll * groups * N && lddt >= heads, "ssm_scan: the rows are too short");
    QI_REQUIRE(state_stride >= (long long)heads * P * N, "ssm_scan: the slots of the state overlap");
    QI_REQUIRE(heads <= 0x7fffffff && n_entries <= 65535, "ssm_scan: grid too large");
    if (n_entries == 0) return 0;
    const dim3 grid(heads, n_entries, (P + kWarps * kCols - 1) / (kWarps * kCols)), block(kWarps * 32);
    const int R = (N + 31) / 32;
    const size_t smem = sizeof(float) * (size_t)kBatch * (2 * (size_t)N + 2 * kWarps * kCols + 2);
#define QI_SCAN(RR)                                                                                                         \
    QI_DISPATCH_DTYPE(dtype, T, {                                                                                           \
        qi::launch(ssm_scan_kernel<T, RR>, grid, block, smem, stream, (const T*)xbc, ldx, (const T*)raw_dt, lddt, dt_bias,     \
                   a_log, d_skip, state, state_stride, y, q_start, start_pos, slot_ids, heads, groups, P, N, write_state);  \
    })
#define QI_END(RR)                                                                                                          \
    QI_DISPATCH_DTYPE(dtype, T, {                                                                                           \
        qi::launch(ssm_end_state_kernel<T, RR>, grid, block, sizeof(float) * ((size_t)kBatch * ((size_t)N + kWarps * kCols + 2) + 1), \
                   stream, (const T*)xbc, ldx, (const T*)raw_dt, lddt, dt_bias, a_log, state, state_stride, q_start, start_pos,  \
                   slot_ids, heads, groups, P, N);                                                                           \
    })
    if (!y && write_state) {          // the end states alone
        if (R <= 1) QI_END(1);
        else if (R <= 2) QI_END(2);
        else if (R <= 4) QI_END(4);
        else QI_END(8);
        return qi::check_launch("ssm_end_state");
    }
    if (R <= 1) QI_SCAN(1);
    else if (R <= 2) QI_SCAN(2);
    else if (R <= 4) QI_SCAN(4);
    else QI_SCAN(8);
#undef QI_SCAN
#undef QI_END
    return qi::check_launch("ssm_scan");
}

// As qi_ssm_scan (y null: the end states alone), a thread or two a channel: for entries of many tokens and N <= 128 (qi_ssm_scan_cols_supported).
extern "C" int qi_ssm_scan_cols_supported(int N) { return N > 0 && N <= 128; }

extern "C" int qi_ssm_scan_cols(const void* xbc, long long ldx, const void* raw_dt, long long lddt, int dtype, const float* dt_bias,
                                const float* a_log, const float* d_skip, float* state, long long state_stride, float* y,
                                const int* q_start, const int* start_pos, const int* slot_ids, int n_entries, int heads,
                                int groups, int P, int N, int write_state, cudaStream_t stream) {
    QI_REQUIRE(n_entries >= 0 && heads > 0 && groups > 0 && P > 0 && qi_ssm_scan_cols_supported(N), "ssm_scan_cols: bad sizes");
    QI_REQUIRE(y || write_state, "ssm_scan_cols: neither outputs nor end states are wanted");
    QI_REQUIRE(heads % groups == 0, "ssm_scan_cols: %d heads are not a multiple of %d groups", heads, groups);
    QI_REQUIRE(ldx >= (long long)heads * P + 2ll * groups * N && lddt >= heads, "ssm_scan_cols: the rows are too short");
    QI_REQUIRE(state_stride >= (long long)heads * P * N, "ssm_scan_cols: the slots of the state overlap");
    QI_REQUIRE(n_entries <= 65535, "ssm_scan_cols: grid too large");
    if (n_entries == 0) return 0;
    const dim3 grid(heads, n_entries, (P + kColChannels - 1) / kColChannels);
#define QI_COLS(NP, SPLIT)                                                                                                 \
    QI_DISPATCH_DTYPE(dtype, T, {                                                                                          \
        if (y) qi::launch(ssm_scan_cols_kernel<T, NP, SPLIT, false>, grid, dim3(kColChannels * SPLIT), 0, stream, (const T*)xbc, ldx, \
                   (const T*)raw_dt, lddt, dt_bias,                                                                        \
                   a_log, d_skip, state, state_stride, y, q_start, start_pos, slot_ids, heads, groups, P, N, write_state,    \
                   vec_ok);                                                                                                \
        else qi::launch(ssm_scan_cols_kernel<T, NP, SPLIT, true>, grid, dim3(kColChannels * SPLIT), 0, stream, (const T*)xbc, ldx, \
                   (const T*)raw_dt, lddt, dt_bias,                                                                        \
                   a_log, d_skip, state, state_stride, y, q_start, start_pos, slot_ids, heads, groups, P, N, write_state,    \
                   vec_ok);                                                                                                \
    })
    // 16-byte loads of B and C: every row, and B's and C's place in it, a multiple of eight numbers from an aligned start
    const int vec_ok = ((uintptr_t)xbc & 15) == 0 && ldx % 8 == 0 && N % 8 == 0 && ((long long)heads * P) % 8 == 0;
    if (N <= 32) QI_COLS(32, 1);
    else if (N <= 64) QI_COLS(64, 2);
    else QI_COLS(128, 2);
#undef QI_COLS
    return qi::check_launch("ssm_scan_cols");
}

// seg_state float32 [segments, heads, P, N] (contiguous); state as for ssm_scan; raw_dt as for ssm_scan; seg_q_start
// [segments + 1]: the segments' first rows; entry_seg [entries + 1]: the entries' first segments; start_pos, slot_ids [entries].
extern "C" int qi_ssm_chain(float* seg_state, float* state, long long state_stride, const void* raw_dt, long long lddt, int dtype,
                            const float* dt_bias, const float* a_log, const int* seg_q_start, const int* entry_seg,
                            const int* start_pos, const int* slot_ids, int n_entries, int max_segments_an_entry, int heads, int P,
                            int N, cudaStream_t stream) {
    QI_REQUIRE(n_entries >= 0 && heads > 0 && P > 0 && N > 0 && max_segments_an_entry >= 0, "ssm_chain: bad sizes");
    QI_REQUIRE(state_stride >= (long long)heads * P * N && lddt >= heads, "ssm_chain: bad layout");
    QI_REQUIRE(n_entries <= 65535 && max_segments_an_entry <= 8192, "ssm_chain: too many entries or segments");
    if (n_entries == 0) return 0;
    QI_DISPATCH_DTYPE(dtype, T, {
        qi::launch(ssm_chain_kernel<T>, dim3(heads, n_entries, (unsigned)(((size_t)P * N + kChainSpan - 1) / kChainSpan)), dim3(256), sizeof(float) * (size_t)(max_segments_an_entry + 1), stream,
                   seg_state, state, state_stride, (const T*)raw_dt, lddt, dt_bias, a_log, seg_q_start, entry_seg, start_pos, slot_ids,
                   heads, P, N);
    });
    return qi::check_launch("ssm_chain");
}

// y float32 [n, width]; z [n, >= width] in z_dtype with `ldz` elements a row; gain float32 [width]; out [n, width] in out_dtype.
// mode 0: rmsnorm_groups(y * silu(z)) * gain; 1: rmsnorm_groups(y) * gain * silu(z); 2: ... * sigmoid(z); 3: ... * z.
extern "C" int qi_group_rmsnorm_gate(const float* y, const void* z, int z_dtype, long long ldz, const float* gain, float eps,
                                     void* out, int out_dtype, int n, int width, int groups, int mode, float out_scale,
                                     cudaStream_t stream) {
    QI_REQUIRE(n >= 0 && width > 0 && groups > 0 && width % groups == 0, "gated_group_rmsnorm: bad sizes n=%d width=%d groups=%d", n, width, groups);
    QI_REQUIRE(ldz >= width && groups <= 65535, "gated_group_rmsnorm: bad layout");
    QI_REQUIRE(mode >= 0 && mode <= 3, "gated_group_rmsnorm: unknown mode %d", mode);
    if (n == 0) return 0;
    const long long n_groups = (long long)n * groups;
    const bool narrow = width / groups <= kNarrowGroup && groups > 1 && (n_groups + 7) / 8 <= 0x7fffffffll;
    QI_DISPATCH_DTYPE(z_dtype, TZ, {
        QI_DISPATCH_DTYPE(out_dtype, TO, {
            if (narrow)
                qi::launch(gated_narrow_group_rmsnorm_kernel<TZ, TO>, dim3((unsigned)((n_groups + 7) / 8)), dim3(256), 0, stream, y,
                           (const TZ*)z, ldz, gain, eps, (TO*)out, n_groups, width, groups, mode, out_scale);
            else
                qi::launch(gated_group_rmsnorm_kernel<TZ, TO>, dim3(n, groups), dim3(256), 0, stream, y, (const TZ*)z, ldz, gain, eps,
                           (TO*)out, width, groups, mode, out_scale);
        });
    });
    return qi::check_launch("gated_group_rmsnorm");
}

extern "C" int qi_gated_group_rmsnorm(const float* y, const void* z, int z_dtype, long long ldz, const float* gain, float eps,
                                      void* out, int out_dtype, int n, int width, int groups, cudaStream_t stream) {
    return qi_group_rmsnorm_gate(y, z, z_dtype, ldz, gain, eps, out, out_dtype, n, width, groups, 0, 1.0f, stream);
}

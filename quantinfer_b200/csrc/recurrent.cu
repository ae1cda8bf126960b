// Recurrent mixers whose state is of fixed size and 32-bit: a gated recurrence per channel (minGRU), and
// recurrences over a matrix state per head that decays and receives the outer product k v^T of every token
// (the time mixing of RWKV with a decay per key channel and a bonus for the current token; lightning
// attention with one constant decay a head; the gated delta rule, whose state is decayed per key channel and corrected
// towards each token's value). Beside them the small kernels these mixers need: the mix of a
// token's input with its predecessor's (token shift) and the weighted sum of two branches' outputs.
//
// All of them work on a step's packed rows: entry e owns rows q_start[e] .. q_start[e + 1] - 1, its first
// token stands at position start_pos[e] of its sequence, its state lies in slot slot_ids[e]. A sequence
// that starts in this step (start_pos 0) takes zeros whatever the slot holds; the state is read at an entry's
// first token and written after its last, so whole prompts, portions cut anywhere and single decode tokens
// run side by side in one launch. Gates, decays, exponentials, the state and all sums are 32-bit; the
// projections' outputs may be bfloat16.
#include "common.cuh"

#include <math.h>

namespace {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x / (1.0f + expf(-x)); }

// ---------------------------------------------------------------------------------------------------
// minGRU:  z = sigmoid(pz + bz), u = px + bx, c = u >= 0 ? u + 1/2 : sigmoid(u)
//          S_t = (1 - z_t) S_(t-1) + z_t c_t            out_t = S_t * silu(pg)
// proj holds pz | px | pg in blocks of `width` columns. The recurrence is linear in S, so an entry of many
// tokens is cut into blockDim.y slices that run side by side: every slice first runs from zero and keeps the
// product of its (1 - z) and its own contribution, the slices' true start states follow by a short chain over
// those pairs in shared memory, and a second pass writes the outputs. With blockDim.y == 1 (steps of single
// tokens) the first pass and the chain fall away.

constexpr int kGruLanes = 32;      // channels a block
constexpr int kGruMaxSlices = 32;
constexpr int kGruAhead = 8;       // tokens whose rows a thread fetches together

template <typename T, typename TO>
__global__ void __launch_bounds__(kGruLanes * kGruMaxSlices)
mingru_scan_kernel(const T* __restrict__ proj, long long ldp, const float* __restrict__ bz, const float* __restrict__ bx,
                   float* __restrict__ state, long long state_stride, TO* __restrict__ out, const int* __restrict__ q_start,
                   const int* __restrict__ start_pos, const int* __restrict__ slot_ids, int width) {
    __shared__ float sh_a[kGruMaxSlices][kGruLanes], sh_b[kGruMaxSlices][kGruLanes];
    qi::pdl_wait();
    const int e = blockIdx.y;
    const int c = blockIdx.x * kGruLanes + threadIdx.x;
    const int slices = blockDim.y, sl = threadIdx.y;
    const int first = q_start[e], len = q_start[e + 1] - first;
    const int per = (len + slices - 1) / slices;
    const int t0 = min(len, sl * per), t1 = min(len, t0 + per);
    const bool live = c < width;
    const float bzc = live ? bz[c] : 0.f, bxc = live ? bx[c] : 0.f;
    float* st = state + (size_t)slot_ids[e] * state_stride + c;
    float S = 0.f;
    // tokens run in groups of kGruAhead whose rows are fetched together, ahead of the arithmetic that depends on S
    if (slices > 1) {
        float a = 1.f, b = 0.f;
        if (live) {
            for (int t = t0; t < t1; t += kGruAhead) {
                float pz[kGruAhead], px[kGruAhead];
#pragma unroll
                for (int i = 0; i < kGruAhead; ++i) {
                    const T* row = proj + (size_t)(first + min(t + i, t1 - 1)) * ldp;
                    pz[i] = qi::to_f32<T>(row[c]);
                    px[i] = qi::to_f32<T>(row[width + c]);
                }
#pragma unroll
                for (int i = 0; i < kGruAhead; ++i) {
                    if (t + i < t1) {
                        const float z = sigmoidf_(pz[i] + bzc);
                        const float u = px[i] + bxc;
                        const float cand = u >= 0.f ? u + 0.5f : sigmoidf_(u);
                        a *= 1.f - z;
                        b = fmaf(1.f - z, b, z * cand);
                    }
                }
            }
        }
        sh_a[sl][threadIdx.x] = a;
        sh_b[sl][threadIdx.x] = b;
        __syncthreads();
    }
    if (!live) return;
    S = start_pos[e] > 0 ? *st : 0.f;
    for (int s = 0; s < sl; ++s) S = fmaf(sh_a[s][threadIdx.x], S, sh_b[s][threadIdx.x]);
    for (int t = t0; t < t1; t += kGruAhead) {
        float pz[kGruAhead], px[kGruAhead], pg[kGruAhead];
#pragma unroll
        for (int i = 0; i < kGruAhead; ++i) {
            const T* row = proj + (size_t)(first + min(t + i, t1 - 1)) * ldp;
            pz[i] = qi::to_f32<T>(row[c]);
            px[i] = qi::to_f32<T>(row[width + c]);
            pg[i] = qi::to_f32<T>(row[2 * width + c]);
        }
#pragma unroll
        for (int i = 0; i < kGruAhead; ++i) {
            if (t + i < t1) {
                const float z = sigmoidf_(pz[i] + bzc);
                const float u = px[i] + bxc;
                const float cand = u >= 0.f ? u + 0.5f : sigmoidf_(u);
                S = fmaf(1.f - z, S, z * cand);
                out[(size_t)(first + t + i) * width + c] = qi::from_f32<TO>(S * siluf_(pg[i]));
            }
        }
    }
    // the slice that holds the entry's last token keeps the state (slices behind it are empty and carry the same value)
    if (sl == slices - 1) *st = S;
}

// ---------------------------------------------------------------------------------------------------
// Token shift: out_s[t] = h[t] + (h[t - 1] - h[t]) * mu_s for s = 0 .. n_mix - 1, h[-1] of an entry's first token
// from the state (the last input of the request's step before; zeros at a sequence's start). One thread per token and
// VEC neighbouring channels (16 bytes where the row length allows); the thread of an entry's first token reads the old
// state and then writes the entry's last input into it, so the state is read and written by one thread in program order.

template <typename T, int VEC>
struct alignas(sizeof(T) * VEC) ShiftPack { T v[VEC]; };

template <typename T, int VEC>
__global__ void __launch_bounds__(256)
token_shift_kernel(const T* __restrict__ h, const float* __restrict__ mu, float* __restrict__ state, long long state_stride,
                   T* __restrict__ out, const int* __restrict__ token_req, const int* __restrict__ q_start,
                   const int* __restrict__ start_pos, const int* __restrict__ slot_ids, int n_tokens, int C, int n_mix) {
    using Pack = ShiftPack<T, VEC>;
    qi::pdl_wait();
    const int per_row = C / VEC;
    const size_t item = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (item >= (size_t)n_tokens * per_row) return;
    const int t = (int)(item / per_row), c = (int)(item % per_row) * VEC;
    const size_t idx = (size_t)t * C + c;
    const int e = token_req[t];
    const int first = q_start[e];
    const Pack xp = *reinterpret_cast<const Pack*>(h + idx);
    float x[VEC], d[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) x[i] = qi::to_f32<T>(xp.v[i]);
    if (t > first) {
        const Pack pp = *reinterpret_cast<const Pack*>(h + idx - C);
#pragma unroll
        for (int i = 0; i < VEC; ++i) d[i] = qi::to_f32<T>(pp.v[i]) - x[i];
    } else {
        float* st = state + (size_t)slot_ids[e] * state_stride + c;
        const bool carried = start_pos[e] > 0;
        const Pack lp = *reinterpret_cast<const Pack*>(h + (size_t)(q_start[e + 1] - 1) * C + c);
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            d[i] = (carried ? st[i] : 0.f) - x[i];
            st[i] = qi::to_f32<T>(lp.v[i]);
        }
    }
    for (int s = 0; s < n_mix; ++s) {
        Pack op;
#pragma unroll
        for (int i = 0; i < VEC; ++i) op.v[i] = qi::from_f32<T>(fmaf(d[i], mu[(size_t)s * C + c + i], x[i]));
        *reinterpret_cast<Pack*>(out + (size_t)s * n_tokens * C + idx) = op;
    }
}

// ---------------------------------------------------------------------------------------------------
// A matrix state per head, S [dk, dv]:
//   mode 0 (decay per key channel, bonus):   o_t = S_(t-1)^T r_t + (sum_i r_i u_i k_i) v_t ;  S_t = diag(w_t) S_(t-1) + k_t v_t^T
//                                            w_t = exp(-exp(lw_t + w0)) from the decay projection's output lw
//   mode 1 (one decay a head, silu inputs):  S_t = lambda S_(t-1) + k_t v_t^T ;  o_t = S_t^T q_t ;  q, k, v = silu of the projections
// A block owns one entry, one head and up to kColThreads value columns; thread j keeps column j of S in registers
// (DK numbers, dk padded with zeros). The operands of kStage tokens are staged in shared memory at a time (decays and
// activations are evaluated there, once a token and channel: thread x stages key channels x, x + kColThreads, ...); in
// the inner loop every thread reads them as broadcasts. The state of a slot is laid out [heads, dv, dk], dk fastest.
//
// The recurrence is linear in S, so long entries are cut into segments that run side by side, as three launches:
// every segment as an entry of its own from zeros, without outputs (o null), leaving its own contribution in a
// scratch row and the product of its decays per key channel in `decay_out`; matrix_state_chain_kernel, which walks an
// entry's segments in order, replaces each contribution by the state its segment starts from and moves the request's
// state to the entry's end; every segment again from that start, now with outputs (write_state 0).

constexpr int kColThreads = 64;

template <typename T, int DK, int MODE>
__global__ void __launch_bounds__(kColThreads, (DK <= 64 ? 8 : 1))
matrix_state_scan_kernel(const T* __restrict__ r, long long ldr, const T* __restrict__ k, long long ldk, const T* __restrict__ v,
                         long long ldv, const T* __restrict__ lw, long long ldw, const float* __restrict__ w0,
                         const float* __restrict__ u, const float* __restrict__ lambda, float* __restrict__ state,
                         long long state_stride, float* __restrict__ o, float* __restrict__ decay_out, int write_state,
                         const int* __restrict__ q_start, const int* __restrict__ start_pos, const int* __restrict__ slot_ids,
                         int heads, int dk, int dv) {
    constexpr int kOwn = (DK + kColThreads - 1) / kColThreads;     // key channels a thread stages
    static_assert(DK % 4 == 0, "the staged operands are read four at a time");
    constexpr int kStage = DK <= 64 ? 8 : 4;                       // tokens a stage
    constexpr int kBonusLanes = kColThreads / kStage;              // threads that share a token's bonus sum
    __shared__ __align__(16) float s_r[kStage][DK], s_k[kStage][DK], s_w[kStage][DK];
    __shared__ float s_v[kStage][kColThreads], s_bonus[kStage], s_u[MODE == 0 ? DK : 1];
    qi::pdl_wait();
    const int hd = blockIdx.x, e = blockIdx.y;
    const int j = blockIdx.z * kColThreads + threadIdx.x;
    const bool live = j < dv;
    const int first = q_start[e], len = q_start[e + 1] - first;
    float* st = state + (size_t)slot_ids[e] * state_stride + ((size_t)hd * dv + (live ? j : 0)) * dk;
    float S[DK];
#pragma unroll
    for (int i = 0; i < DK; ++i) S[i] = 0.f;
    // a column is dk numbers in a row: 16 bytes a load where the column starts on such a boundary
    const bool wide = dk % 4 == 0 && (reinterpret_cast<size_t>(st) & 15) == 0;
    if (live && start_pos[e] > 0) {
        if (wide) {
#pragma unroll
            for (int i = 0; i < DK; i += 4)
                if (i < dk) {
                    const float4 x = *reinterpret_cast<const float4*>(st + i);
                    S[i] = x.x, S[i + 1] = x.y, S[i + 2] = x.z, S[i + 3] = x.w;
                }
        } else {
#pragma unroll
            for (int i = 0; i < DK; ++i) if (i < dk) S[i] = st[i];
        }
    }
    const float lam = MODE == 1 ? lambda[hd] : 0.f;
    float w0r[kOwn], dsum[kOwn];        // dsum: minus the logarithm of the product of this entry's decays
#pragma unroll
    for (int m = 0; m < kOwn; ++m) {
        const int i = threadIdx.x + m * kColThreads;
        const bool in = MODE == 0 && i < dk;
        w0r[m] = in ? w0[(size_t)hd * dk + i] : 0.f;
        dsum[m] = 0.f;
    }
    if (MODE == 0)
        for (int i = threadIdx.x; i < DK; i += kColThreads) s_u[i] = i < dk ? u[(size_t)hd * dk + i] : 0.f;
    // A stage's numbers are fetched into registers one stage ahead, while the stage before is worked through.
    T f_r[kOwn][kStage], f_k[kOwn][kStage], f_w[MODE == 0 ? kOwn : 1][kStage], f_v[kStage];
    auto fetch = [&](int base) {
        const int nt = min(kStage, len - base);
#pragma unroll
        for (int m = 0; m < kOwn; ++m) {
            const int i = threadIdx.x + m * kColThreads;
            const bool in = i < dk;
#pragma unroll
            for (int tt = 0; tt < kStage; ++tt) {
                if (in && tt < nt) {
                    const size_t row = (size_t)(first + base + tt);
                    f_r[m][tt] = r[row * ldr + (size_t)hd * dk + i];
                    f_k[m][tt] = k[row * ldk + (size_t)hd * dk + i];
                    if (MODE == 0) f_w[m][tt] = lw[row * ldw + (size_t)hd * dk + i];
                }
            }
        }
#pragma unroll
        for (int tt = 0; tt < kStage; ++tt)
            if (live && tt < nt) f_v[tt] = v[(size_t)(first + base + tt) * ldv + (size_t)hd * dv + j];
    };
    if (len > 0) fetch(0);
    for (int base = 0; base < len; base += kStage) {
        const int nt = min(kStage, len - base);
        __syncthreads();
#pragma unroll
        for (int m = 0; m < kOwn; ++m) {
            const int i = threadIdx.x + m * kColThreads;
            if (i < DK) {
                const bool in = i < dk;
#pragma unroll
                for (int tt = 0; tt < kStage; ++tt) {
                    if (tt < nt) {
                        float rv = 0.f, kv = 0.f, wv = 0.f;
                        if (in) {
                            rv = qi::to_f32<T>(f_r[m][tt]);
                            kv = qi::to_f32<T>(f_k[m][tt]);
                            if (MODE == 0) {
                                const float rate = expf(qi::to_f32<T>(f_w[m][tt]) + w0r[m]);
                                wv = expf(-rate);
                                dsum[m] += rate;
                            } else {
                                rv = siluf_(rv);
                                kv = siluf_(kv);
                            }
                        }
                        s_r[tt][i] = rv;
                        s_k[tt][i] = kv;
                        if (MODE == 0) s_w[tt][i] = wv;
                    }
                }
            }
        }
#pragma unroll
        for (int tt = 0; tt < kStage; ++tt) {
            if (tt < nt) {
                float vv = live ? qi::to_f32<T>(f_v[tt]) : 0.f;
                if (MODE == 1) vv = siluf_(vv);
                s_v[tt][threadIdx.x] = vv;
            }
        }
        if (base + kStage < len) fetch(base + kStage);
        if (MODE == 0 && o) {
            __syncthreads();
            // the bonus of the current token, sum_i r_i u_i k_i: kBonusLanes threads a token, each every kBonusLanes-th channel
            const int tt = threadIdx.x / kBonusLanes, sub = threadIdx.x % kBonusLanes;
            float b = 0.f;
            if (tt < nt)
                for (int i = sub; i < DK; i += kBonusLanes) b = fmaf(s_r[tt][i] * s_u[i], s_k[tt][i], b);
#pragma unroll
            for (int d = kBonusLanes / 2; d > 0; d >>= 1) b += __shfl_xor_sync(0xffffffffu, b, d);
            if (sub == 0) s_bonus[tt] = b;
        }
        __syncthreads();
        // every thread reads the staged operands as broadcasts, four key channels an instruction
        if (!o) {                       // a segment's own contribution only
            for (int tt = 0; tt < nt; ++tt) {
                const float vj = s_v[tt][threadIdx.x];
                const float4* k4 = reinterpret_cast<const float4*>(s_k[tt]);
                const float4* w4 = reinterpret_cast<const float4*>(s_w[tt]);
#pragma unroll
                for (int i = 0; i < DK; i += 4) {
                    const float4 kk = k4[i >> 2];
                    const float4 ww = MODE == 0 ? w4[i >> 2] : make_float4(lam, lam, lam, lam);
                    S[i] = fmaf(ww.x, S[i], kk.x * vj);
                    S[i + 1] = fmaf(ww.y, S[i + 1], kk.y * vj);
                    S[i + 2] = fmaf(ww.z, S[i + 2], kk.z * vj);
                    S[i + 3] = fmaf(ww.w, S[i + 3], kk.w * vj);
                }
            }
            continue;
        }
        for (int tt = 0; tt < nt; ++tt) {
            const float vj = s_v[tt][threadIdx.x];
            const float4* r4 = reinterpret_cast<const float4*>(s_r[tt]);
            const float4* k4 = reinterpret_cast<const float4*>(s_k[tt]);
            const float4* w4 = reinterpret_cast<const float4*>(s_w[tt]);
            float acc4[4] = {0.f, 0.f, 0.f, 0.f};
            if (MODE == 0) {
#pragma unroll
                for (int i = 0; i < DK; i += 4) {
                    const float4 rr = r4[i >> 2], kk = k4[i >> 2], ww = w4[i >> 2];
                    acc4[0] = fmaf(rr.x, S[i], acc4[0]);
                    S[i] = fmaf(ww.x, S[i], kk.x * vj);
                    acc4[1] = fmaf(rr.y, S[i + 1], acc4[1]);
                    S[i + 1] = fmaf(ww.y, S[i + 1], kk.y * vj);
                    acc4[2] = fmaf(rr.z, S[i + 2], acc4[2]);
                    S[i + 2] = fmaf(ww.z, S[i + 2], kk.z * vj);
                    acc4[3] = fmaf(rr.w, S[i + 3], acc4[3]);
                    S[i + 3] = fmaf(ww.w, S[i + 3], kk.w * vj);
                }
            } else {
#pragma unroll
                for (int i = 0; i < DK; i += 4) {
                    const float4 rr = r4[i >> 2], kk = k4[i >> 2];
                    S[i] = fmaf(lam, S[i], kk.x * vj);
                    acc4[0] = fmaf(rr.x, S[i], acc4[0]);
                    S[i + 1] = fmaf(lam, S[i + 1], kk.y * vj);
                    acc4[1] = fmaf(rr.y, S[i + 1], acc4[1]);
                    S[i + 2] = fmaf(lam, S[i + 2], kk.z * vj);
                    acc4[2] = fmaf(rr.z, S[i + 2], acc4[2]);
                    S[i + 3] = fmaf(lam, S[i + 3], kk.w * vj);
                    acc4[3] = fmaf(rr.w, S[i + 3], acc4[3]);
                }
            }
            float acc = (acc4[0] + acc4[1]) + (acc4[2] + acc4[3]);
            if (MODE == 0) acc = fmaf(s_bonus[tt], vj, acc);
            if (live) o[(size_t)(first + base + tt) * ((size_t)heads * dv) + (size_t)hd * dv + j] = acc;
        }
    }
    if (live && write_state) {
        if (wide) {
#pragma unroll
            for (int i = 0; i < DK; i += 4)
                if (i < dk) *reinterpret_cast<float4*>(st + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
        } else {
#pragma unroll
            for (int i = 0; i < DK; ++i) if (i < dk) st[i] = S[i];
        }
    }
    if (decay_out && blockIdx.z == 0) {
        float all = 1.f;
        if (MODE == 1) for (int t = 0; t < len; ++t) all *= lam;
#pragma unroll
        for (int m = 0; m < kOwn; ++m) {
            const int i = threadIdx.x + m * kColThreads;
            if (i < dk) decay_out[((size_t)e * heads + hd) * dk + i] = MODE == 0 ? expf(-dsum[m]) : all;
        }
    }
}

// Between the two passes over segments: seg_state [segments, heads, dv, dk] holds every segment's own contribution and
// receives the state the segment starts from; seg_decay [segments, heads, dk] the product of each segment's decays.
// Entry e owns segments entry_seg[e] .. entry_seg[e + 1] - 1; its request's state moves to the entry's end. A thread
// owns one element of a head's matrix and fetches kChainAhead segments' numbers at a time, so that the walk waits for
// memory once a group and not once a segment.
constexpr int kChainThreads = 256, kChainAhead = 8;

__global__ void __launch_bounds__(kChainThreads)
matrix_state_chain_kernel(float* __restrict__ seg_state, const float* __restrict__ seg_decay, float* __restrict__ state,
                          long long state_stride, const int* __restrict__ entry_seg, const int* __restrict__ start_pos,
                          const int* __restrict__ slot_ids, int heads, int dk, int dv) {
    qi::pdl_wait();
    const int hd = blockIdx.x, e = blockIdx.y;
    const int elems = dk * dv;
    const int el = blockIdx.z * kChainThreads + threadIdx.x;
    if (el >= elems) return;
    const int s0 = entry_seg[e], s1 = entry_seg[e + 1];
    float* st = state + (size_t)slot_ids[e] * state_stride + (size_t)hd * elems + el;
    float S = start_pos[e] > 0 ? *st : 0.f;
    const size_t seg_stride = (size_t)heads * elems, dec_stride = (size_t)heads * dk;
    float* row = seg_state + ((size_t)s0 * heads + hd) * elems + el;
    const float* dec = seg_decay + ((size_t)s0 * heads + hd) * dk + el % dk;
    for (int s = s0; s < s1; s += kChainAhead) {
        float own[kChainAhead], d[kChainAhead];
#pragma unroll
        for (int a = 0; a < kChainAhead; ++a) {
            const bool in = s + a < s1;
            own[a] = in ? row[a * seg_stride] : 0.f;
            d[a] = in ? dec[a * dec_stride] : 1.f;
        }
#pragma unroll
        for (int a = 0; a < kChainAhead; ++a) {
            if (s + a < s1) {
                row[a * seg_stride] = S;
                S = fmaf(d[a], S, own[a]);
            }
        }
        row += kChainAhead * seg_stride;
        dec += kChainAhead * dec_stride;
    }
    *st = S;
}

// out = sa * (a_0 + a_1 + ...) + sb * (b_0 + b_1 + ...), 32-bit, for the next norm's fused addition: a and b each come
// whole or as the partial sums of a product whose contraction was split (ka, kb parts of n numbers, added in order).
template <typename TA, typename TB>
__global__ void scaled_sum_kernel(const TA* __restrict__ a, int ka, const TB* __restrict__ b, int kb, float sa, float sb,
                                  float* __restrict__ out, size_t n) {
    qi::pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
        float x = qi::to_f32<TA>(a[idx]), y = qi::to_f32<TB>(b[idx]);
        for (int p = 1; p < ka; ++p) x += qi::to_f32<TA>(a[(size_t)p * n + idx]);
        for (int p = 1; p < kb; ++p) y += qi::to_f32<TB>(b[(size_t)p * n + idx]);
        out[idx] = fmaf(sa, x, sb * y);
    }
}

}  // namespace

// proj [n, >= 3 width] in `dtype` (z | x | g, `ldp` elements a row); bz, bx float32 [width]; state float32, one row of
// `width` numbers a slot, `state_stride` floats apart; out [n, width] in `out_dtype`; slices: 1 .. 32, how many parts an
// entry is cut into (1 for steps of single tokens).
extern "C" int qi_mingru_scan(const void* proj, long long ldp, int dtype, const float* bz, const float* bx, float* state,
                              long long state_stride, void* out, int out_dtype, const int* q_start, const int* start_pos,
                              const int* slot_ids, int n_entries, int width, int slices, cudaStream_t stream) {
    QI_REQUIRE(n_entries >= 0 && width > 0 && ldp >= 3ll * width && state_stride >= width, "mingru_scan: bad sizes");
    QI_REQUIRE(slices >= 1 && slices <= kGruMaxSlices, "mingru_scan: %d slices are outside 1..%d", slices, kGruMaxSlices);
    QI_REQUIRE(n_entries <= 65535, "mingru_scan: grid too large");
    if (n_entries == 0) return 0;
    const dim3 grid((width + kGruLanes - 1) / kGruLanes, n_entries), block(kGruLanes, slices);
    QI_DISPATCH_DTYPE(dtype, T, {
        QI_DISPATCH_DTYPE(out_dtype, TO, {
            qi::launch(mingru_scan_kernel<T, TO>, grid, block, 0, stream, (const T*)proj, ldp, bz, bx, state, state_stride, (TO*)out,
                       q_start, start_pos, slot_ids, width);
        });
    });
    return qi::check_launch("mingru_scan");
}

// h [n, C] in `dtype`; mu float32 [n_mix, C]; state float32, C numbers a slot; out [n_mix, n, C] in `dtype`.
extern "C" int qi_token_shift(const void* h, int dtype, const float* mu, float* state, long long state_stride, void* out,
                              const int* token_req, const int* q_start, const int* start_pos, const int* slot_ids, int n_tokens,
                              int channels, int n_mix, cudaStream_t stream) {
    QI_REQUIRE(n_tokens >= 0 && channels > 0 && n_mix > 0 && state_stride >= channels, "token_shift: bad sizes");
    if (n_tokens == 0) return 0;
    QI_DISPATCH_DTYPE(dtype, T, {
        constexpr int kVec = 16 / (int)sizeof(T);
        const bool wide = channels % kVec == 0 && (((uintptr_t)h | (uintptr_t)out) & 15) == 0;
        const size_t total = (size_t)n_tokens * (wide ? channels / kVec : channels);
        QI_REQUIRE((total + 255) / 256 <= 0x7fffffffull, "token_shift: grid too large");
        if (wide)
            qi::launch(token_shift_kernel<T, kVec>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, (const T*)h, mu, state,
                       state_stride, (T*)out, token_req, q_start, start_pos, slot_ids, n_tokens, channels, n_mix);
        else
            qi::launch(token_shift_kernel<T, 1>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, (const T*)h, mu, state,
                       state_stride, (T*)out, token_req, q_start, start_pos, slot_ids, n_tokens, channels, n_mix);
    });
    return qi::check_launch("token_shift");
}

extern "C" int qi_matrix_state_scan_supported(int dk) { return dk > 0 && dk <= 256; }

// mode 0: r, k, lw [n, >= heads dk], v [n, >= heads dv] in `dtype` (each with its own row stride); w0, u float32
// [heads dk]; lambda unused. mode 1: r (the queries), k, v the same; lambda float32 [heads]; lw, w0, u unused.
// state float32 [heads, dv, dk] a slot, `state_stride` floats apart; o float32 [n, heads dv], or null: no outputs
// (a segment's own contribution is all that is wanted). decay_out (or null): float32 [n_entries, heads, dk], receives
// the product of each entry's decays per key channel. write_state 0: the state is read, not written.
extern "C" int qi_matrix_state_scan(int mode, const void* r, long long ldr, const void* k, long long ldk, const void* v, long long ldv,
                                    const void* lw, long long ldw, int dtype, const float* w0, const float* u, const float* lambda,
                                    float* state, long long state_stride, float* o, float* decay_out, int write_state,
                                    const int* q_start, const int* start_pos, const int* slot_ids, int n_entries, int heads,
                                    int dk, int dv, cudaStream_t stream) {
    QI_REQUIRE(mode == 0 || mode == 1, "matrix_state_scan: unknown mode %d", mode);
    QI_REQUIRE(n_entries >= 0 && heads > 0 && dv > 0 && qi_matrix_state_scan_supported(dk), "matrix_state_scan: bad sizes (keys of 1..256)");
    QI_REQUIRE(ldr >= (long long)heads * dk && ldk >= (long long)heads * dk && ldv >= (long long)heads * dv, "matrix_state_scan: the rows are too short");
    QI_REQUIRE(mode == 1 || (lw && w0 && u && ldw >= (long long)heads * dk), "matrix_state_scan: the decay's operands are missing");
    QI_REQUIRE(mode == 0 || lambda, "matrix_state_scan: the heads' decays are missing");
    QI_REQUIRE(state_stride >= (long long)heads * dk * dv, "matrix_state_scan: the slots of the state overlap");
    QI_REQUIRE(o || write_state, "matrix_state_scan: neither outputs nor the state are wanted");
    QI_REQUIRE(n_entries <= 65535 && (dv + kColThreads - 1) / kColThreads <= 65535, "matrix_state_scan: grid too large");
    if (n_entries == 0) return 0;
    const dim3 grid(heads, n_entries, (dv + kColThreads - 1) / kColThreads), block(kColThreads);
#define QI_MS(DKP, MODE)                                                                                                        \
    qi::launch(matrix_state_scan_kernel<T, DKP, MODE>, grid, block, 0, stream, (const T*)r, ldr, (const T*)k, ldk, (const T*)v, ldv, \
               (const T*)lw, ldw, w0, u, lambda, state, state_stride, o, decay_out, write_state, q_start, start_pos, slot_ids, heads, dk, dv)
#define QI_MS_DK(MODE)                              \
    if (dk <= 16) QI_MS(16, MODE);                  \
    else if (dk <= 32) QI_MS(32, MODE);             \
    else if (dk <= 64) QI_MS(64, MODE);             \
    else if (dk <= 128) QI_MS(128, MODE);           \
    else QI_MS(256, MODE)
    QI_DISPATCH_DTYPE(dtype, T, {
        if (mode == 0) { QI_MS_DK(0); } else { QI_MS_DK(1); }
    });
#undef QI_MS_DK
#undef QI_MS
    return qi::check_launch("matrix_state_scan");
}

// seg_state float32 [segments, heads, dv, dk]; seg_decay float32 [segments, heads, dk]; state float32 [heads, dv, dk] a
// slot; entry_seg [n_entries + 1].
// Blocks of the scan kernel (mode, key size, operand type) that one SM holds at a time, or 0 when it cannot be told:
// whoever cuts long entries into segments sizes them so that the launch fills whole waves.
extern "C" int qi_matrix_state_scan_blocks_per_sm(int mode, int dk, int dtype) {
    if ((mode != 0 && mode != 1) || !qi_matrix_state_scan_supported(dk) || (dtype != qi::kF32 && dtype != qi::kBF16)) return 0;
    int blocks = 0;
#define QI_MS_OCC(DKP, MODE) cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, matrix_state_scan_kernel<T, DKP, MODE>, kColThreads, 0)
#define QI_MS_OCC_DK(MODE)                          \
    if (dk <= 16) QI_MS_OCC(16, MODE);              \
    else if (dk <= 32) QI_MS_OCC(32, MODE);         \
    else if (dk <= 64) QI_MS_OCC(64, MODE);         \
    else if (dk <= 128) QI_MS_OCC(128, MODE);       \
    else QI_MS_OCC(256, MODE)
    QI_DISPATCH_DTYPE(dtype, T, {
        if (mode == 0) { QI_MS_OCC_DK(0); } else { QI_MS_OCC_DK(1); }
    });
#undef QI_MS_OCC_DK
#undef QI_MS_OCC
    if (cudaGetLastError() != cudaSuccess) return 0;
    return blocks;
}

extern "C" int qi_matrix_state_chain(float* seg_state, const float* seg_decay, float* state, long long state_stride,
                                     const int* entry_seg, const int* start_pos, const int* slot_ids, int n_entries, int heads,
                                     int dk, int dv, cudaStream_t stream) {
    QI_REQUIRE(n_entries >= 0 && heads > 0 && dk > 0 && dv > 0, "matrix_state_chain: bad sizes");
    QI_REQUIRE(state_stride >= (long long)heads * dk * dv, "matrix_state_chain: the slots of the state overlap");
    QI_REQUIRE(n_entries <= 65535, "matrix_state_chain: grid too large");
    if (n_entries == 0) return 0;
    qi::launch(matrix_state_chain_kernel, dim3(heads, n_entries, (dk * dv + kChainThreads - 1) / kChainThreads), dim3(kChainThreads), 0, stream, seg_state,
               seg_decay, state, state_stride, entry_seg, start_pos, slot_ids, heads, dk, dv);
    return qi::check_launch("matrix_state_chain");
}

// a [ka, n] in `dtype_a`, b [kb, n] in `dtype_b` (parts n numbers apart); out float32 [n].
extern "C" int qi_scaled_sum(const void* a, int ka, int dtype_a, const void* b, int kb, int dtype_b, float sa, float sb, float* out,
                             long long n, cudaStream_t stream) {
    QI_REQUIRE(n >= 0 && ka >= 1 && kb >= 1, "scaled_sum: bad sizes");
    if (n == 0) return 0;
    size_t blocks = ((size_t)n + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    QI_DISPATCH_DTYPE(dtype_a, TA, {
        QI_DISPATCH_DTYPE(dtype_b, TB, {
            qi::launch(scaled_sum_kernel<TA, TB>, dim3((unsigned)blocks), dim3(256), 0, stream, (const TA*)a, ka, (const TB*)b, kb, sa, sb,
                       out, (size_t)n);
        });
    });
    return qi::check_launch("scaled_sum");
}

namespace {

// ---------------------------------------------------------------------------------------------------
// The gated delta rule over a matrix state per head, S [dk, dv]:
//     S' = diag(w_t) S_(t-1) ;  u_t = beta_t (v_t - S'^T k_t) ;  S_t = S' + k_t u_t^T ;  o_t = S_t^T q_t
// with q and k made unit vectors per head (x / sqrt(sum x^2 + unit_eps)), q times q_scale, beta_t = sigmoid(b_t),
// w_t = exp(-exp(A_h) softplus(lw_t + w0)) per head and key channel; heads / qk_heads value heads share a head of q and k.
//
// The factor on the state is not diagonal, so a long entry cannot be cut into segments as the recurrences above are; but
// every column of S (one value channel) moves on its own, and what a token costs on the way from S_(t-1) to S_t is one
// sum over the key channels. So a column is spread over kDeltaOwn-channel parts held by neighbouring lanes, which add
// their partial sums with shuffles: a token is 2 x kDeltaOwn dependent multiply-adds and log2(lanes) shuffles long
// instead of 2 x dk, and a block of kDeltaThreads threads owns an entry, a head and kDeltaThreads / lanes columns, so
// that a prompt of one request still spreads over heads x dv / columns blocks. The operands of kStage tokens are
// staged in shared memory at a time (unit vectors' factors, beta, softplus and both exponentials are evaluated there,
// once a token and channel, in 32-bit) from registers that were loaded a stage ahead. The read-out's sum lies off the
// path from one token's state to the next.
constexpr int kDeltaThreads = 128;

// A load that stays where it is written: the compiler may move a plain load of read-only memory down to its first
// use, which would undo fetching a stage ahead.
template <typename T> __device__ __forceinline__ T load_now(const T* p);
template <> __device__ __forceinline__ float load_now<float>(const float* p) {
    float v;
    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}
template <> __device__ __forceinline__ qi::bf16 load_now<qi::bf16>(const qi::bf16* p) {
    unsigned short v;
    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return __ushort_as_bfloat16(v);
}

template <typename T, int DK, int OWN>
__global__ void __launch_bounds__(kDeltaThreads)
delta_rule_scan_kernel(const T* __restrict__ q, long long ldq, const T* __restrict__ k, long long ldk, const T* __restrict__ v,
                       long long ldv, const T* __restrict__ lw, long long ldw, const T* __restrict__ bproj, long long ldb,
                       const float* __restrict__ w0, const float* __restrict__ a_log, float* __restrict__ state,
                       long long state_stride, float* __restrict__ o, int write_state, const int* __restrict__ q_start,
                       const int* __restrict__ start_pos, const int* __restrict__ slot_ids, int heads, int qk_heads, int dk, int dv,
                       float unit_eps, float q_scale) {
    static_assert((OWN == 4 || OWN == 8) && DK % OWN == 0, "a column is cut into parts of four or eight channels");
    constexpr int kGroups = OWN / 4;                       // groups of four neighbouring channels a thread keeps
    constexpr int kLanes = DK / OWN;                       // lanes that share a column (a power of two, at most 32)
    constexpr int kCols = kDeltaThreads / kLanes;          // columns a block owns
    constexpr int kStage = DK <= 128 ? 8 : 4;              // tokens a stage
    constexpr int kItems = (DK * kStage + kDeltaThreads - 1) / kDeltaThreads;    // (token, channel) pairs a thread stages
    constexpr int kVItems = (kCols * kStage + kDeltaThreads - 1) / kDeltaThreads;
    constexpr int kNormLanes = kDeltaThreads / kStage;     // threads that share a token's two sums of squares
    static_assert(kLanes >= 1 && kLanes <= 32 && kNormLanes <= 32, "sizes of the staging");
    __shared__ __align__(16) float s_q[kStage][DK], s_k[kStage][DK], s_w[kStage][DK];
    __shared__ float s_v[kStage][kCols];
    __shared__ __align__(16) float4 s_tok[kStage];        // a token's numbers: factor of the unit key, of the unit query, beta
    qi::pdl_wait();
    const int hd = blockIdx.x, e = blockIdx.y;
    const int hq = hd / (heads / qk_heads);
    const int part = threadIdx.x % kLanes, col = threadIdx.x / kLanes;
    const int j = blockIdx.z * kCols + col;
    const bool live = j < dv;
    const int first = q_start[e], len = q_start[e + 1] - first;
    // this thread's channels: group g holds four neighbours at g * (DK / groups) + 4 * part, so that neighbouring lanes read
    // neighbouring 16 bytes of the staged operands
    int ch[kGroups];
#pragma unroll
    for (int g = 0; g < kGroups; ++g) ch[g] = g * (DK / kGroups) + part * 4;
    float* st = state + (size_t)slot_ids[e] * state_stride + ((size_t)hd * dv + (live ? j : 0)) * dk;
    float S[OWN];
#pragma unroll
    for (int i = 0; i < OWN; ++i) S[i] = 0.f;
    const bool wide = dk % 4 == 0 && (reinterpret_cast<size_t>(st) & 15) == 0;
    auto move_state = [&](bool store) {
#pragma unroll
        for (int g = 0; g < kGroups; ++g) {
            const int c = ch[g];
            if (wide && c + 3 < dk) {
                float4* p = reinterpret_cast<float4*>(st + c);
                if (store) *p = make_float4(S[4 * g], S[4 * g + 1], S[4 * g + 2], S[4 * g + 3]);
                else { const float4 x = *p; S[4 * g] = x.x, S[4 * g + 1] = x.y, S[4 * g + 2] = x.z, S[4 * g + 3] = x.w; }
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (c + i < dk) { if (store) st[c + i] = S[4 * g + i]; else S[4 * g + i] = st[c + i]; }
            }
        }
    };
    if (live && start_pos[e] > 0) move_state(false);
    const float rate = expf(a_log[hd]);
    // a stage's numbers are fetched into registers one stage ahead, while the stage before is worked through
    T f_q[kItems], f_k[kItems], f_w[kItems], f_v[kVItems], f_b = qi::from_f32<T>(0.f);
    float w0r[kItems];
#pragma unroll
    for (int m = 0; m < kItems; ++m) {
        const int i = (threadIdx.x + m * kDeltaThreads) % DK;
        w0r[m] = i < dk ? w0[(size_t)hd * dk + i] : 0.f;
        f_q[m] = f_k[m] = f_w[m] = qi::from_f32<T>(0.f);
    }
#pragma unroll
    for (int m = 0; m < kVItems; ++m) f_v[m] = qi::from_f32<T>(0.f);
    auto fetch = [&](int base) {
        const int nt = min(kStage, len - base);
#pragma unroll
        for (int m = 0; m < kItems; ++m) {
            const int idx = threadIdx.x + m * kDeltaThreads, tt = idx / DK, i = idx % DK;
            if (tt < nt && i < dk) {
                const size_t row = (size_t)(first + base + tt);
                f_q[m] = load_now<T>(q + row * ldq + (size_t)hq * dk + i);
                f_k[m] = load_now<T>(k + row * ldk + (size_t)hq * dk + i);
                f_w[m] = load_now<T>(lw + row * ldw + (size_t)hd * dk + i);
            }
        }
#pragma unroll
        for (int m = 0; m < kVItems; ++m) {
            const int idx = threadIdx.x + m * kDeltaThreads, tt = idx / kCols, c = idx % kCols;
            if (tt < nt && blockIdx.z * kCols + c < dv) f_v[m] = load_now<T>(v + (size_t)(first + base + tt) * ldv + (size_t)hd * dv + blockIdx.z * kCols + c);
        }
        if ((int)threadIdx.x < nt) f_b = load_now<T>(bproj + (size_t)(first + base + threadIdx.x) * ldb + hd);
    };
    if (len > 0) fetch(0);
    for (int base = 0; base < len; base += kStage) {
        const int nt = min(kStage, len - base);
        __syncthreads();
#pragma unroll
        for (int m = 0; m < kItems; ++m) {
            const int idx = threadIdx.x + m * kDeltaThreads, tt = idx / DK, i = idx % DK;
            if (tt < nt) {
                float qv = 0.f, kv = 0.f, wv = 0.f;
                if (i < dk) {
                    qv = qi::to_f32<T>(f_q[m]);
                    kv = qi::to_f32<T>(f_k[m]);
                    const float x = qi::to_f32<T>(f_w[m]) + w0r[m];
                    wv = expf(-rate * (x > 20.f ? x : log1pf(expf(x))));          // softplus
                }
                s_q[tt][i] = qv;
                s_k[tt][i] = kv;
                s_w[tt][i] = wv;
            }
        }
#pragma unroll
        for (int m = 0; m < kVItems; ++m) {
            const int idx = threadIdx.x + m * kDeltaThreads, tt = idx / kCols, c = idx % kCols;
            if (idx < kCols * kStage && tt < nt) s_v[tt][c] = blockIdx.z * kCols + c < dv ? qi::to_f32<T>(f_v[m]) : 0.f;
        }
        // a token's numbers, one float4: the factors of the unit key and of the unit query come below, beta here
        if ((int)threadIdx.x < nt) s_tok[threadIdx.x].z = sigmoidf_(qi::to_f32<T>(f_b));
        if (base + kStage < len) fetch(base + kStage);
        __syncthreads();
        {   // the lengths of a token's q and k: kNormLanes threads a token, each every kNormLanes-th channel
            const int tt = threadIdx.x / kNormLanes, sub = threadIdx.x % kNormLanes;
            float sq = 0.f, sk = 0.f;
            if (tt < nt)
                for (int i = sub; i < DK; i += kNormLanes) {
                    sq = fmaf(s_q[tt][i], s_q[tt][i], sq);
                    sk = fmaf(s_k[tt][i], s_k[tt][i], sk);
                }
#pragma unroll
            for (int d = kNormLanes / 2; d > 0; d >>= 1) {
                sq += __shfl_xor_sync(0xffffffffu, sq, d);
                sk += __shfl_xor_sync(0xffffffffu, sk, d);
            }
            if (sub == 0 && tt < nt) {
                s_tok[tt].x = 1.0f / sqrtf(sk + unit_eps);
                s_tok[tt].y = q_scale / sqrtf(sq + unit_eps);
            }
        }
        __syncthreads();
        // one token after the other; the next token's operands are read while this one's sums are on their way
        float4 kk[kGroups], gg[kGroups], rr[kGroups], tok = s_tok[0];
        float vj = s_v[0][col];
#pragma unroll
        for (int g = 0; g < kGroups; ++g) {
            kk[g] = *reinterpret_cast<const float4*>(&s_k[0][ch[g]]);
            gg[g] = *reinterpret_cast<const float4*>(&s_w[0][ch[g]]);
            rr[g] = *reinterpret_cast<const float4*>(&s_q[0][ch[g]]);
        }
#pragma unroll
        for (int tt = 0; tt < kStage; ++tt) {
            if (tt >= nt) break;             // (the same for the whole block; what was read ahead of the last token is not used)
            float4 kn[kGroups], gn[kGroups], rn[kGroups], tokn = tok;
            float vn = vj;
            if (tt + 1 < kStage) {
                tokn = s_tok[tt + 1];
                vn = s_v[tt + 1][col];
#pragma unroll
                for (int g = 0; g < kGroups; ++g) {
                    kn[g] = *reinterpret_cast<const float4*>(&s_k[tt + 1][ch[g]]);
                    gn[g] = *reinterpret_cast<const float4*>(&s_w[tt + 1][ch[g]]);
                    rn[g] = *reinterpret_cast<const float4*>(&s_q[tt + 1][ch[g]]);
                }
            }
            // the decay, and what the decayed state holds for this key
            float held = 0.f;
#pragma unroll
            for (int g = 0; g < kGroups; ++g) {
                S[4 * g] *= gg[g].x; S[4 * g + 1] *= gg[g].y; S[4 * g + 2] *= gg[g].z; S[4 * g + 3] *= gg[g].w;
                const float pa = fmaf(kk[g].y, S[4 * g + 1], kk[g].x * S[4 * g]), pb = fmaf(kk[g].w, S[4 * g + 3], kk[g].z * S[4 * g + 2]);
                held += pa + pb;
            }
#pragma unroll
            for (int d = kLanes / 2; d > 0; d >>= 1) held += __shfl_xor_sync(0xffffffffu, held, d);
            const float uk = tok.z * (vj - held * tok.x) * tok.x;        // the correction, times the factor of the unit key
            float acc = 0.f;
#pragma unroll
            for (int g = 0; g < kGroups; ++g) {
                S[4 * g] = fmaf(kk[g].x, uk, S[4 * g]); S[4 * g + 1] = fmaf(kk[g].y, uk, S[4 * g + 1]);
                S[4 * g + 2] = fmaf(kk[g].z, uk, S[4 * g + 2]); S[4 * g + 3] = fmaf(kk[g].w, uk, S[4 * g + 3]);
                const float pa = fmaf(rr[g].y, S[4 * g + 1], rr[g].x * S[4 * g]), pb = fmaf(rr[g].w, S[4 * g + 3], rr[g].z * S[4 * g + 2]);
                acc += pa + pb;
            }
            if (o) {
#pragma unroll
                for (int d = kLanes / 2; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
                if (live && part == 0) o[(size_t)(first + base + tt) * ((size_t)heads * dv) + (size_t)hd * dv + j] = acc * tok.y;
            }
            if (tt + 1 < kStage) {
                tok = tokn, vj = vn;
#pragma unroll
                for (int g = 0; g < kGroups; ++g) kk[g] = kn[g], gg[g] = gn[g], rr[g] = rn[g];
            }
        }
    }
    if (live && write_state) move_state(true);
}


// The same recurrence for steps with prompt portions, in two launches. The blocks of one head would each evaluate the
// same unit vectors, softplus and exponentials; so a first kernel, a block a token, writes them once, in 32-bit: the
// unit queries (times q_scale) and unit keys [n, qk_heads, DK], the decays [n, heads, DK] (rows padded with zeros to
// the kernel's key size DK, so that every row starts on a 16-byte boundary) and beta [n, heads]. The scan then only
// moves rows: 16 bytes a cp.async into one of two buffers, a stage ahead of the tokens that are worked through.
template <typename T>
__global__ void __launch_bounds__(128)
delta_prepare_kernel(const T* __restrict__ q, long long ldq, const T* __restrict__ k, long long ldk, const T* __restrict__ lw,
                     long long ldw, const T* __restrict__ bproj, long long ldb, const float* __restrict__ w0,
                     const float* __restrict__ a_log, float* __restrict__ qn, float* __restrict__ kn, float* __restrict__ wn,
                     float* __restrict__ beta, int heads, int qk_heads, int dk, int DK, float unit_eps, float q_scale) {
    qi::pdl_wait();
    const size_t t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int h = warp; h < 2 * qk_heads; h += 4) {          // a warp a head of q or of k
        const bool is_q = h < qk_heads;
        const int hh = is_q ? h : h - qk_heads;
        const T* src = (is_q ? q + t * ldq : k + t * ldk) + (size_t)hh * dk;
        float ss = 0.f;
        for (int i = lane; i < dk; i += 32) {
            const float x = qi::to_f32<T>(src[i]);
            ss = fmaf(x, x, ss);
        }
        ss = qi::warp_sum(ss);
        const float f = (is_q ? q_scale : 1.0f) / sqrtf(ss + unit_eps);
        float* dst = (is_q ? qn : kn) + (t * qk_heads + hh) * DK;
        for (int i = lane; i < DK; i += 32) dst[i] = i < dk ? qi::to_f32<T>(src[i]) * f : 0.f;
    }
    for (int idx = threadIdx.x; idx < heads * DK; idx += blockDim.x) {
        const int hd = idx / DK, i = idx % DK;
        float w = 0.f;
        if (i < dk) {
            const float x = qi::to_f32<T>(lw[t * ldw + (size_t)hd * dk + i]) + w0[(size_t)hd * dk + i];
            w = expf(-expf(a_log[hd]) * (x > 20.f ? x : log1pf(expf(x))));          // softplus
        }
        wn[t * heads * DK + idx] = w;
    }
    for (int hd = threadIdx.x; hd < heads; hd += blockDim.x) beta[t * heads + hd] = sigmoidf_(qi::to_f32<T>(bproj[t * ldb + hd]));
}

__device__ __forceinline__ void copy16_async(void* smem_dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src) : "memory");
}

template <typename T, int DK>
__global__ void __launch_bounds__(kDeltaThreads)
delta_rule_stream_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ wn,
                         const float* __restrict__ beta, const T* __restrict__ v, long long ldv, float* __restrict__ state,
                         long long state_stride, float* __restrict__ o, int write_state, const int* __restrict__ q_start,
                         const int* __restrict__ start_pos, const int* __restrict__ slot_ids, int heads, int qk_heads, int dk, int dv) {
    constexpr int OWN = 8, kGroups = 2;
    constexpr int kLanes = DK / OWN, kCols = kDeltaThreads / kLanes;
    constexpr int kStage = DK <= 128 ? 8 : 4;
    constexpr int kChunks = (kStage * DK / 4 + kDeltaThreads - 1) / kDeltaThreads;     // 16-byte pieces of an operand a thread copies a stage
    constexpr int kVItems = (kCols * kStage + kDeltaThreads - 1) / kDeltaThreads;
    __shared__ __align__(16) float s_q[2][kStage][DK], s_k[2][kStage][DK], s_w[2][kStage][DK];
    __shared__ float s_v[2][kStage][kCols], s_beta[2][kStage];
    qi::pdl_wait();
    const int hd = blockIdx.x, e = blockIdx.y;
    const int hq = hd / (heads / qk_heads);
    const int part = threadIdx.x % kLanes, col = threadIdx.x / kLanes;
    const int j = blockIdx.z * kCols + col;
    const bool live = j < dv;
    const int first = q_start[e], len = q_start[e + 1] - first;
    int ch[kGroups];
#pragma unroll
    for (int g = 0; g < kGroups; ++g) ch[g] = g * (DK / kGroups) + part * 4;
    float* st = state + (size_t)slot_ids[e] * state_stride + ((size_t)hd * dv + (live ? j : 0)) * dk;
    float S[OWN];
#pragma unroll
    for (int i = 0; i < OWN; ++i) S[i] = 0.f;
    const bool wide = dk % 4 == 0 && (reinterpret_cast<size_t>(st) & 15) == 0;
    auto move_state = [&](bool store) {
#pragma unroll
        for (int g = 0; g < kGroups; ++g) {
            const int c = ch[g];
            if (wide && c + 3 < dk) {
                float4* p = reinterpret_cast<float4*>(st + c);
                if (store) *p = make_float4(S[4 * g], S[4 * g + 1], S[4 * g + 2], S[4 * g + 3]);
                else { const float4 x = *p; S[4 * g] = x.x, S[4 * g + 1] = x.y, S[4 * g + 2] = x.z, S[4 * g + 3] = x.w; }
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (c + i < dk) { if (store) st[c + i] = S[4 * g + i]; else S[4 * g + i] = st[c + i]; }
            }
        }
    };
    if (live && start_pos[e] > 0) move_state(false);
    T f_v[kVItems];
    float f_b = 0.f;
#pragma unroll
    for (int m = 0; m < kVItems; ++m) f_v[m] = qi::from_f32<T>(0.f);
    // q, k and the decays of a stage: asynchronous copies into buffer `buf`; values and beta: into registers
    auto request = [&](int base, int buf) {
        const int nt = min(kStage, len - base);
#pragma unroll
        for (int m = 0; m < kChunks; ++m) {
            const int c = threadIdx.x + m * kDeltaThreads, tt = c / (DK / 4), piece = c % (DK / 4);
            if (tt < nt) {
                const size_t row = (size_t)(first + base + tt);
                copy16_async(&s_q[buf][tt][piece * 4], qn + (row * qk_heads + hq) * DK + piece * 4);
                copy16_async(&s_k[buf][tt][piece * 4], kn + (row * qk_heads + hq) * DK + piece * 4);
                copy16_async(&s_w[buf][tt][piece * 4], wn + (row * heads + hd) * DK + piece * 4);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
#pragma unroll
        for (int m = 0; m < kVItems; ++m) {
            const int idx = threadIdx.x + m * kDeltaThreads, tt = idx / kCols, c = idx % kCols;
            if (tt < nt && blockIdx.z * kCols + c < dv) f_v[m] = load_now<T>(v + (size_t)(first + base + tt) * ldv + (size_t)hd * dv + blockIdx.z * kCols + c);
        }
        if ((int)threadIdx.x < nt) f_b = load_now<float>(beta + (size_t)(first + base + threadIdx.x) * heads + hd);
    };
    if (len > 0) request(0, 0);
    int buf = 0;
    for (int base = 0; base < len; base += kStage, buf ^= 1) {
        const int nt = min(kStage, len - base);
        // this stage's values and beta leave the registers before the next stage's are requested into them
#pragma unroll
        for (int m = 0; m < kVItems; ++m) {
            const int idx = threadIdx.x + m * kDeltaThreads, tt = idx / kCols, c = idx % kCols;
            if (idx < kCols * kStage && tt < nt) s_v[buf][tt][c] = blockIdx.z * kCols + c < dv ? qi::to_f32<T>(f_v[m]) : 0.f;
        }
        if ((int)threadIdx.x < nt) s_beta[buf][threadIdx.x] = f_b;
        if (base + kStage < len) {
            request(base + kStage, buf ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        float4 kk[kGroups], gg[kGroups], rr[kGroups];
        float vj = s_v[buf][0][col], bt = s_beta[buf][0];
#pragma unroll
        for (int g = 0; g < kGroups; ++g) {
            kk[g] = *reinterpret_cast<const float4*>(&s_k[buf][0][ch[g]]);
            gg[g] = *reinterpret_cast<const float4*>(&s_w[buf][0][ch[g]]);
            rr[g] = *reinterpret_cast<const float4*>(&s_q[buf][0][ch[g]]);
        }
#pragma unroll
        for (int tt = 0; tt < kStage; ++tt) {
            if (tt >= nt) break;             // (the same for the whole block; what was read ahead of the last token is not used)
            float4 kx[kGroups], gx[kGroups], rx[kGroups];
            float vn = vj, bn = bt;
            if (tt + 1 < kStage) {
                vn = s_v[buf][tt + 1][col];
                bn = s_beta[buf][tt + 1];
#pragma unroll
                for (int g = 0; g < kGroups; ++g) {
                    kx[g] = *reinterpret_cast<const float4*>(&s_k[buf][tt + 1][ch[g]]);
                    gx[g] = *reinterpret_cast<const float4*>(&s_w[buf][tt + 1][ch[g]]);
                    rx[g] = *reinterpret_cast<const float4*>(&s_q[buf][tt + 1][ch[g]]);
                }
            }
            float held = 0.f;
#pragma unroll
            for (int g = 0; g < kGroups; ++g) {
                S[4 * g] *= gg[g].x; S[4 * g + 1] *= gg[g].y; S[4 * g + 2] *= gg[g].z; S[4 * g + 3] *= gg[g].w;
                const float pa = fmaf(kk[g].y, S[4 * g + 1], kk[g].x * S[4 * g]), pb = fmaf(kk[g].w, S[4 * g + 3], kk[g].z * S[4 * g + 2]);
                held += pa + pb;
            }
#pragma unroll
            for (int d = kLanes / 2; d > 0; d >>= 1) held += __shfl_xor_sync(0xffffffffu, held, d);
            const float uk = bt * (vj - held);
            float acc = 0.f;
#pragma unroll
            for (int g = 0; g < kGroups; ++g) {
                S[4 * g] = fmaf(kk[g].x, uk, S[4 * g]); S[4 * g + 1] = fmaf(kk[g].y, uk, S[4 * g + 1]);
                S[4 * g + 2] = fmaf(kk[g].z, uk, S[4 * g + 2]); S[4 * g + 3] = fmaf(kk[g].w, uk, S[4 * g + 3]);
                const float pa = fmaf(rr[g].y, S[4 * g + 1], rr[g].x * S[4 * g]), pb = fmaf(rr[g].w, S[4 * g + 3], rr[g].z * S[4 * g + 2]);
                acc += pa + pb;
            }
            if (o) {
#pragma unroll
                for (int d = kLanes / 2; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
                if (live && part == 0) o[(size_t)(first + base + tt) * ((size_t)heads * dv) + (size_t)hd * dv + j] = acc;
            }
            if (tt + 1 < kStage) {
                vj = vn, bt = bn;
#pragma unroll
                for (int g = 0; g < kGroups; ++g) kk[g] = kx[g], gg[g] = gx[g], rr[g] = rx[g];
            }
        }
        __syncthreads();        // everyone is done with this buffer before the stage after next is requested into it
    }
    if (live && write_state) move_state(true);
}

}  // namespace

extern "C" int qi_delta_rule_scan_supported(int dk) { return dk > 0 && dk <= 256; }

// q (the queries) and k [n, >= qk_heads dk], v [n, >= heads dv], lw [n, >= heads dk] (the decay projection's output), bproj
// [n, >= heads] (beta's logits), all in `dtype`, each with its own row stride; w0 float32 [heads dk] (added to lw); a_log
// float32 [heads] (the logarithm of each head's rate); state float32 [heads, dv, dk] a slot, `state_stride` floats apart;
// o float32 [n, heads dv] or null (the state moves on and nothing else is written); write_state 0: the state is only read.
// scratch (or null): float32, qi_delta_rule_scratch_floats(n_tokens, ...) numbers; when given, the recurrence runs in its
// two-launch form for steps with prompt portions (the same sums; the unit vectors' factors are applied before them instead of after).
extern "C" long long qi_delta_rule_scratch_floats(int n_tokens, int heads, int qk_heads, int dk) {
    const long long DKP = dk <= 16 ? 16 : dk <= 32 ? 32 : dk <= 64 ? 64 : dk <= 128 ? 128 : 256;
    return (long long)n_tokens * ((2ll * qk_heads + heads) * DKP + heads);
}

extern "C" int qi_delta_rule_scan(const void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv,
                                  const void* lw, long long ldw, const void* bproj, long long ldb, int dtype, const float* w0,
                                  const float* a_log, float* state, long long state_stride, float* o, int write_state,
                                  const int* q_start, const int* start_pos, const int* slot_ids, int n_entries, int heads,
                                  int qk_heads, int dk, int dv, float unit_eps, float q_scale, float* scratch, int n_tokens,
                                  cudaStream_t stream) {
    QI_REQUIRE(n_entries >= 0 && heads > 0 && dv > 0 && qi_delta_rule_scan_supported(dk), "delta_rule_scan: bad sizes (keys of 1..256)");
    QI_REQUIRE(qk_heads > 0 && heads % qk_heads == 0, "delta_rule_scan: %d heads are not a multiple of %d heads of q and k", heads, qk_heads);
    QI_REQUIRE(ldq >= (long long)qk_heads * dk && ldk >= (long long)qk_heads * dk && ldv >= (long long)heads * dv &&
               ldw >= (long long)heads * dk && ldb >= heads, "delta_rule_scan: the rows are too short");
    QI_REQUIRE(q && k && v && lw && bproj && w0 && a_log && unit_eps > 0.f, "delta_rule_scan: an operand is missing");
    QI_REQUIRE(state_stride >= (long long)heads * dk * dv, "delta_rule_scan: the slots of the state overlap");
    QI_REQUIRE(o || write_state, "delta_rule_scan: neither outputs nor the state are wanted");
    QI_REQUIRE(n_entries <= 65535, "delta_rule_scan: grid too large");
    if (n_entries == 0) return 0;
    if (scratch) {          // steps with prompt portions: unit vectors, decays and beta once a token, then a scan that only moves rows
        const int DKP = dk <= 16 ? 16 : dk <= 32 ? 32 : dk <= 64 ? 64 : dk <= 128 ? 128 : 256;
        QI_REQUIRE(n_tokens > 0 && n_tokens <= 0x7fffffff / 4, "delta_rule_scan: bad token count");
        float* qn = scratch;
        float* kn = qn + (size_t)n_tokens * qk_heads * DKP;
        float* wn = kn + (size_t)n_tokens * qk_heads * DKP;
        float* bt = wn + (size_t)n_tokens * heads * DKP;
        QI_DISPATCH_DTYPE(dtype, T, {
            qi::launch(delta_prepare_kernel<T>, dim3(n_tokens), dim3(128), 0, stream, (const T*)q, ldq, (const T*)k, ldk, (const T*)lw, ldw,
                       (const T*)bproj, ldb, w0, a_log, qn, kn, wn, bt, heads, qk_heads, dk, DKP, unit_eps, q_scale);
        });
        if (int rc = qi::check_launch("delta_rule_prepare")) return rc;
#define QI_DS(DKC)                                                                                                                      \
    do {                                                                                                                                \
        constexpr int cols = kDeltaThreads / (DKC / 8);                                                                                 \
        qi::launch(delta_rule_stream_kernel<T, DKC>, dim3(heads, n_entries, (dv + cols - 1) / cols), dim3(kDeltaThreads), 0, stream, qn, kn, wn, \
                   bt, (const T*)v, ldv, state, state_stride, o, write_state, q_start, start_pos, slot_ids, heads, qk_heads, dk, dv);   \
    } while (0)
        QI_DISPATCH_DTYPE(dtype, T, {
            if (DKP == 16) QI_DS(16);
            else if (DKP == 32) QI_DS(32);
            else if (DKP == 64) QI_DS(64);
            else if (DKP == 128) QI_DS(128);
            else QI_DS(256);
        });
#undef QI_DS
        return qi::check_launch("delta_rule_stream");
    }
#define QI_DR(DKP, OWN)                                                                                                             \
    do {                                                                                                                            \
        constexpr int cols = kDeltaThreads / (DKP / OWN);                                                                           \
        qi::launch(delta_rule_scan_kernel<T, DKP, OWN>, dim3(heads, n_entries, (dv + cols - 1) / cols), dim3(kDeltaThreads), 0, stream, \
                   (const T*)q, ldq, (const T*)k, ldk, (const T*)v, ldv, (const T*)lw, ldw, (const T*)bproj, ldb, w0, a_log, state,  \
                   state_stride, o, write_state, q_start, start_pos, slot_ids, heads, qk_heads, dk, dv, unit_eps, q_scale);         \
    } while (0)
    // (four channels a thread where keys are short, eight else: with four everywhere the blocks of a head, twice as many,
    // spent more on staging the same operands than the shorter sums saved: 1,032 us against 850 for 2,048 tokens of 16 heads)
    QI_DISPATCH_DTYPE(dtype, T, {
        if (dk <= 8) QI_DR(8, 4);
        else if (dk <= 16) QI_DR(16, 4);
        else if (dk <= 32) QI_DR(32, 8);
        else if (dk <= 64) QI_DR(64, 8);
        else if (dk <= 128) QI_DR(128, 8);
        else QI_DR(256, 8);
    });
#undef QI_DR
    return qi::check_launch("delta_rule_scan");
}

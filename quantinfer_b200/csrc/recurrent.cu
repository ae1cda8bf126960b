// Recurrent mixers whose state is of fixed size and 32-bit: a gated recurrence per channel (minGRU), and
// recurrences over a matrix state per head that decays and receives the outer product k v^T of every token
// (the time mixing of RWKV with a decay per key channel and a bonus for the current token; lightning
// attention with one constant decay a head). Beside them the small kernels these mixers need: the mix of a
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
    if (slices > 1) {
        float a = 1.f, b = 0.f;
        if (live) {
            for (int t = t0; t < t1; ++t) {
                const T* row = proj + (size_t)(first + t) * ldp;
                const float z = sigmoidf_(qi::to_f32<T>(row[c]) + bzc);
                const float u = qi::to_f32<T>(row[width + c]) + bxc;
                const float cand = u >= 0.f ? u + 0.5f : sigmoidf_(u);
                a *= 1.f - z;
                b = fmaf(1.f - z, b, z * cand);
            }
        }
        sh_a[sl][threadIdx.x] = a;
        sh_b[sl][threadIdx.x] = b;
        __syncthreads();
    }
    if (!live) return;
    S = start_pos[e] > 0 ? *st : 0.f;
    for (int s = 0; s < sl; ++s) S = fmaf(sh_a[s][threadIdx.x], S, sh_b[s][threadIdx.x]);
    for (int t = t0; t < t1; ++t) {
        const T* row = proj + (size_t)(first + t) * ldp;
        const float z = sigmoidf_(qi::to_f32<T>(row[c]) + bzc);
        const float u = qi::to_f32<T>(row[width + c]) + bxc;
        const float cand = u >= 0.f ? u + 0.5f : sigmoidf_(u);
        S = fmaf(1.f - z, S, z * cand);
        out[(size_t)(first + t) * width + c] = qi::from_f32<TO>(S * siluf_(qi::to_f32<T>(row[2 * width + c])));
    }
    // the slice that holds the entry's last token keeps the state (slices behind it are empty and carry the same value)
    if (sl == slices - 1) *st = S;
}

// ---------------------------------------------------------------------------------------------------
// Token shift: out_s[t] = h[t] + (h[t - 1] - h[t]) * mu_s for s = 0 .. n_mix - 1, h[-1] of an entry's first token
// from the state (the last input of the request's step before; zeros at a sequence's start). One thread per
// (token, channel); the thread of an entry's first token reads the old state and then writes the entry's last
// input into it, so the state is read and written by one thread in program order.

template <typename T>
__global__ void __launch_bounds__(256)
token_shift_kernel(const T* __restrict__ h, const float* __restrict__ mu, float* __restrict__ state, long long state_stride,
                   T* __restrict__ out, const int* __restrict__ token_req, const int* __restrict__ q_start,
                   const int* __restrict__ start_pos, const int* __restrict__ slot_ids, int n_tokens, int C, int n_mix) {
    qi::pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n_tokens * C) return;
    const int t = (int)(idx / C), c = (int)(idx % C);
    const int e = token_req[t];
    const int first = q_start[e];
    const float x = qi::to_f32<T>(h[idx]);
    float prev;
    if (t > first) {
        prev = qi::to_f32<T>(h[idx - C]);
    } else {
        float* st = state + (size_t)slot_ids[e] * state_stride + c;
        prev = start_pos[e] > 0 ? *st : 0.f;
        *st = qi::to_f32<T>(h[(size_t)(q_start[e + 1] - 1) * C + c]);
    }
    const float d = prev - x;
    for (int s = 0; s < n_mix; ++s) out[(size_t)s * n_tokens * C + idx] = qi::from_f32<T>(fmaf(d, mu[(size_t)s * C + c], x));
}

// ---------------------------------------------------------------------------------------------------
// A matrix state per head, S [dk, dv]:
//   mode 0 (decay per key channel, bonus):   o_t = S_(t-1)^T r_t + (sum_i r_i u_i k_i) v_t ;  S_t = diag(w_t) S_(t-1) + k_t v_t^T
//                                            w_t = exp(-exp(lw_t + w0)) from the decay projection's output lw
//   mode 1 (one decay a head, silu inputs):  S_t = lambda S_(t-1) + k_t v_t^T ;  o_t = S_t^T q_t ;  q, k, v = silu of the projections
// A block owns one entry, one head and up to kColThreads value columns; thread j keeps column j of S in registers
// (DK numbers, dk padded with zeros). The operands of kStage tokens are staged in shared memory at a time (decays and
// activations are evaluated there, once a token and channel); in the inner loop every thread reads them as broadcasts.
// The state of a slot is laid out [heads, dv, dk], dk fastest.

constexpr int kColThreads = 64;
constexpr int kStage = 8;

template <typename T, int DK, int MODE>
__global__ void __launch_bounds__(kColThreads)
matrix_state_scan_kernel(const T* __restrict__ r, long long ldr, const T* __restrict__ k, long long ldk, const T* __restrict__ v,
                         long long ldv, const T* __restrict__ lw, long long ldw, const float* __restrict__ w0,
                         const float* __restrict__ u, const float* __restrict__ lambda, float* __restrict__ state,
                         long long state_stride, float* __restrict__ o, const int* __restrict__ q_start,
                         const int* __restrict__ start_pos, const int* __restrict__ slot_ids, int heads, int dk, int dv) {
    __shared__ float s_r[kStage][DK], s_k[kStage][DK], s_w[kStage][DK], s_v[kStage][kColThreads], s_bonus[kStage];
    qi::pdl_wait();
    const int hd = blockIdx.x, e = blockIdx.y;
    const int j = blockIdx.z * kColThreads + threadIdx.x;
    const bool live = j < dv;
    const int first = q_start[e], len = q_start[e + 1] - first;
    float* st = state + (size_t)slot_ids[e] * state_stride + ((size_t)hd * dv + (live ? j : 0)) * dk;
    float S[DK];
#pragma unroll
    for (int i = 0; i < DK; ++i) S[i] = 0.f;
    if (live && start_pos[e] > 0) {
#pragma unroll
        for (int i = 0; i < DK; ++i) if (i < dk) S[i] = st[i];
    }
    const float lam = MODE == 1 ? lambda[hd] : 0.f;
    for (int base = 0; base < len; base += kStage) {
        const int nt = min(kStage, len - base);
        __syncthreads();
        for (int idx = threadIdx.x; idx < nt * DK; idx += kColThreads) {
            const int tt = idx / DK, i = idx % DK;
            const size_t row = (size_t)(first + base + tt);
            float rv = 0.f, kv = 0.f, wv = 0.f;
            if (i < dk) {
                rv = qi::to_f32<T>(r[row * ldr + (size_t)hd * dk + i]);
                kv = qi::to_f32<T>(k[row * ldk + (size_t)hd * dk + i]);
                if (MODE == 0) {
                    wv = expf(-expf(qi::to_f32<T>(lw[row * ldw + (size_t)hd * dk + i]) + w0[(size_t)hd * dk + i]));
                } else {
                    rv = siluf_(rv);
                    kv = siluf_(kv);
                }
            }
            s_r[tt][i] = rv;
            s_k[tt][i] = kv;
            if (MODE == 0) s_w[tt][i] = wv;
        }
        for (int idx = threadIdx.x; idx < nt * kColThreads; idx += kColThreads) {
            const int tt = idx / kColThreads, jj = blockIdx.z * kColThreads + idx % kColThreads;
            float vv = 0.f;
            if (jj < dv) {
                vv = qi::to_f32<T>(v[(size_t)(first + base + tt) * ldv + (size_t)hd * dv + jj]);
                if (MODE == 1) vv = siluf_(vv);
            }
            s_v[tt][idx % kColThreads] = vv;
        }
        if (MODE == 0) {
            __syncthreads();
            if (threadIdx.x < nt) {     // the bonus of the current token: sum_i r_i u_i k_i, in the order of i
                float b = 0.f;
                for (int i = 0; i < dk; ++i) b = fmaf(s_r[threadIdx.x][i] * u[(size_t)hd * dk + i], s_k[threadIdx.x][i], b);
                s_bonus[threadIdx.x] = b;
            }
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float vj = s_v[tt][threadIdx.x];
            float acc = 0.f;
            if (MODE == 0) {
#pragma unroll
                for (int i = 0; i < DK; ++i) {
                    acc = fmaf(s_r[tt][i], S[i], acc);
                    S[i] = fmaf(s_w[tt][i], S[i], s_k[tt][i] * vj);
                }
                acc = fmaf(s_bonus[tt], vj, acc);
            } else {
#pragma unroll
                for (int i = 0; i < DK; ++i) {
                    S[i] = fmaf(lam, S[i], s_k[tt][i] * vj);
                    acc = fmaf(s_r[tt][i], S[i], acc);
                }
            }
            if (live) o[(size_t)(first + base + tt) * ((size_t)heads * dv) + (size_t)hd * dv + j] = acc;
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < DK; ++i) if (i < dk) st[i] = S[i];
    }
}

// out = sa * a + sb * b, 32-bit, for the next norm's fused addition.
template <typename T>
__global__ void scaled_sum_kernel(const T* __restrict__ a, const T* __restrict__ b, float sa, float sb, float* __restrict__ out, size_t n) {
    qi::pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x)
        out[idx] = fmaf(sa, qi::to_f32<T>(a[idx]), sb * qi::to_f32<T>(b[idx]));
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
    const size_t total = (size_t)n_tokens * channels;
    QI_REQUIRE((total + 255) / 256 <= 0x7fffffffull, "token_shift: grid too large");
    QI_DISPATCH_DTYPE(dtype, T, {
        qi::launch(token_shift_kernel<T>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, (const T*)h, mu, state,
                   state_stride, (T*)out, token_req, q_start, start_pos, slot_ids, n_tokens, channels, n_mix);
    });
    return qi::check_launch("token_shift");
}

extern "C" int qi_matrix_state_scan_supported(int dk) { return dk > 0 && dk <= 256; }

// mode 0: r, k, lw [n, >= heads dk], v [n, >= heads dv] in `dtype` (each with its own row stride); w0, u float32
// [heads dk]; lambda unused. mode 1: r (the queries), k, v the same; lambda float32 [heads]; lw, w0, u unused.
// state float32 [heads, dv, dk] a slot, `state_stride` floats apart; o float32 [n, heads dv].
extern "C" int qi_matrix_state_scan(int mode, const void* r, long long ldr, const void* k, long long ldk, const void* v, long long ldv,
                                    const void* lw, long long ldw, int dtype, const float* w0, const float* u, const float* lambda,
                                    float* state, long long state_stride, float* o, const int* q_start, const int* start_pos,
                                    const int* slot_ids, int n_entries, int heads, int dk, int dv, cudaStream_t stream) {
    QI_REQUIRE(mode == 0 || mode == 1, "matrix_state_scan: unknown mode %d", mode);
    QI_REQUIRE(n_entries >= 0 && heads > 0 && dv > 0 && qi_matrix_state_scan_supported(dk), "matrix_state_scan: bad sizes (keys of 1..256)");
    QI_REQUIRE(ldr >= (long long)heads * dk && ldk >= (long long)heads * dk && ldv >= (long long)heads * dv, "matrix_state_scan: the rows are too short");
    QI_REQUIRE(mode == 1 || (lw && w0 && u && ldw >= (long long)heads * dk), "matrix_state_scan: the decay's operands are missing");
    QI_REQUIRE(mode == 0 || lambda, "matrix_state_scan: the heads' decays are missing");
    QI_REQUIRE(state_stride >= (long long)heads * dk * dv, "matrix_state_scan: the slots of the state overlap");
    QI_REQUIRE(n_entries <= 65535 && (dv + kColThreads - 1) / kColThreads <= 65535, "matrix_state_scan: grid too large");
    if (n_entries == 0) return 0;
    const dim3 grid(heads, n_entries, (dv + kColThreads - 1) / kColThreads), block(kColThreads);
#define QI_MS(DKP, MODE)                                                                                                        \
    qi::launch(matrix_state_scan_kernel<T, DKP, MODE>, grid, block, 0, stream, (const T*)r, ldr, (const T*)k, ldk, (const T*)v, ldv, \
               (const T*)lw, ldw, w0, u, lambda, state, state_stride, o, q_start, start_pos, slot_ids, heads, dk, dv)
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

// a, b [n] in `dtype`; out float32 [n].
extern "C" int qi_scaled_sum(const void* a, const void* b, int dtype, float sa, float sb, float* out, long long n, cudaStream_t stream) {
    QI_REQUIRE(n >= 0, "scaled_sum: bad size");
    if (n == 0) return 0;
    size_t blocks = ((size_t)n + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    QI_DISPATCH_DTYPE(dtype, T, {
        qi::launch(scaled_sum_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, (const T*)a, (const T*)b, sa, sb, out, (size_t)n);
    });
    return qi::check_launch("scaled_sum");
}

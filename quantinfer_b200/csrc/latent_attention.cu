// Attention over a cached low-rank latent, in the form that never expands keys and values.
//
// A position caches one row [c (R numbers) | kr (r numbers)]: the normalised latent and a rotated key
// part that all heads share. Per head h the key would be k_h = Wk_h c and the value v_h = Wv_h c. With
// the query's plain part moved into the latent space, ql_h = Wk_h^T q_h, the score of query i and key j is
//
//     s_ij = (ql_h(i) . c(j) + qr_h(i) . kr(j)) * scale
//
// and the output is Wv_h (sum_j p_ij c(j)); so every head reads the same rows, with a query of width
// W = R + r and a "value" that is the row's first R numbers. The two per-head products (into the latent
// space and out of it) are batched matrix products outside these kernels.
//
//     lo = 0, or i - window + 1 for a windowed layer;   j runs over lo .. i
//     p_ij = exp(s_ij - m) / (sum_j exp(s_ij - m) + exp(sink_h - m))      (sink: optional, one number a head,
//                                                                          no key, no value, not scaled)
//
// qi_latent_prepare: per token, from the row of the fused projection [q heads | latent projection]:
// rotates each head's r-part into the query buffer, and (when the layer projects its own latent)
// normalises the latent (32-bit, gain per coordinate), rotates the shared key part and writes the row
// into the paged cache. Rotation: pair i of the first `rot_dims` coordinates of the part, (2i, 2i + 1) or, when
// `half_split`, (i, i + rot_dims / 2), turns by the angle position * inv_freq[i], computed here in 32-bit (no
// table, so no limit on positions); cos and sin are multiplied by `magnitude` (1 for the plain rotation).
//
// qi_latent_attention_generic: 32-bit arithmetic for any sizes; one block per (token, head).
#include "common.cuh"

#include <math.h>

namespace {

template <typename TP, typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const TP* __restrict__ proj, long long ldp, int kv_off, T* __restrict__ q_out,
                      const float* __restrict__ gain, float eps, const float* __restrict__ inv_freq, int rot_dims,
                      const int* __restrict__ positions, const int* __restrict__ token_req,
                      const int* __restrict__ block_table, int max_blocks, int page_size, int num_pages,
                      T* __restrict__ cache, int H, int d, int r, int R, int half_split, float magnitude,
                      int* __restrict__ status) {
    extern __shared__ float smem[];
    float* cs = smem;                 // [rot_dims / 2]
    float* sn = smem + rot_dims / 2;  // [rot_dims / 2]
    float* scratch = sn + rot_dims / 2;   // [32]
    qi::pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    for (int i = threadIdx.x; i < rot_dims / 2; i += blockDim.x) {
        const float a = (float)pos * inv_freq[i];
        float s, c;
        sincosf(a, &s, &c);
        cs[i] = c * magnitude;
        sn[i] = s * magnitude;
    }
    __syncthreads();
    const TP* row = proj + (size_t)t * ldp;
    const int W = R + r;
    // the rotated part of every head's query
    for (int idx = threadIdx.x; idx < H * r; idx += blockDim.x) {
        const int h = idx / r, j = idx % r;
        const TP* part = row + (size_t)h * (d + r) + d;
        float v;
        if (j < rot_dims) {
            const int half = rot_dims >> 1;
            const int i = half_split ? (j < half ? j : j - half) : j >> 1;
            const bool second = half_split ? j >= half : (j & 1);
            const float a = qi::to_f32<TP>(part[half_split ? i : 2 * i]), b = qi::to_f32<TP>(part[half_split ? i + half : 2 * i + 1]);
            v = second ? b * cs[i] + a * sn[i] : a * cs[i] - b * sn[i];
        } else {
            v = qi::to_f32<TP>(part[j]);
        }
        q_out[((size_t)t * H + h) * W + R + j] = qi::from_f32<T>(v);
    }
    if (kv_off < 0) return;
    const TP* z = row + kv_off;
    float ss = 0.f;
    for (int i = threadIdx.x; i < R; i += blockDim.x) {
        const float v = qi::to_f32<TP>(z[i]);
        ss = fmaf(v, v, ss);
    }
    ss = qi::block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)R + eps);
    const int page = block_table[(size_t)token_req[t] * max_blocks + pos / page_size];
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0 && status) atomicOr(status, qi::kStatusBadPage);
        return;
    }
    T* dst = cache + ((size_t)page * page_size + pos % page_size) * W;
    for (int i = threadIdx.x; i < R; i += blockDim.x) dst[i] = qi::from_f32<T>(qi::to_f32<TP>(z[i]) * inv * gain[i]);
    for (int j = threadIdx.x; j < r; j += blockDim.x) {
        float v;
        if (j < rot_dims) {
            const int half = rot_dims >> 1;
            const int i = half_split ? (j < half ? j : j - half) : j >> 1;
            const bool second = half_split ? j >= half : (j & 1);
            const float a = qi::to_f32<TP>(z[R + (half_split ? i : 2 * i)]), b = qi::to_f32<TP>(z[R + (half_split ? i + half : 2 * i + 1)]);
            v = second ? b * cs[i] + a * sn[i] : a * cs[i] - b * sn[i];
        } else {
            v = qi::to_f32<TP>(z[R + j]);
        }
        dst[R + j] = qi::from_f32<T>(v);
    }
}

constexpr int kWarps = 4;
constexpr int kMaxR = 512;
constexpr int kAccPerLane = kMaxR / 32;

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
latent_attention_generic_kernel(const T* __restrict__ q, T* __restrict__ out, const T* __restrict__ cache,
                                const float* __restrict__ sink, const int* __restrict__ block_table, int max_blocks,
                                int page_size, int num_pages, const int* __restrict__ positions,
                                const int* __restrict__ token_req, int H, int W, int R, float scale, int window,
                                int* __restrict__ status) {
    extern __shared__ float smem[];
    float* q_s = smem;                          // [W]
    float* part_acc = smem + W;                 // [kWarps][R]
    float* part_m = part_acc + kWarps * R;      // [kWarps]
    float* part_l = part_m + kWarps;            // [kWarps]

    qi::pdl_wait();
    const int t = blockIdx.y, h = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = positions[t];
    const int* table = block_table + (size_t)token_req[t] * max_blocks;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

    const T* qrow = q + ((size_t)t * H + h) * W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) q_s[i] = qi::to_f32<T>(qrow[i]);
    __syncthreads();

    float m = -INFINITY, l = 0.f;
    float acc[kAccPerLane];
#pragma unroll
    for (int i = 0; i < kAccPerLane; ++i) acc[i] = 0.f;

    bool bad_page = false;
    for (int base = lo + warp * 32; base <= pos; base += kWarps * 32) {
        const int j = base + lane;
        float s = -INFINITY;
        if (j <= pos) {
            const int page = table[j / page_size];
            if (page < 0 || page >= num_pages) {
                bad_page = true;
            } else {
                const T* krow = cache + ((size_t)page * page_size + (j % page_size)) * (size_t)W;
                float dot = 0.f;
                for (int i = 0; i < W; ++i) dot = fmaf(q_s[i], qi::to_f32<T>(krow[i]), dot);
                s = dot * scale;
            }
        }
        const float cm = qi::warp_max(s);
        if (cm == -INFINITY) continue;  // only after a bad page
        const float m_new = fmaxf(m, cm);
        const float corr = expf(m - m_new);  // m = -inf on the first chunk gives 0
        const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
        l = l * corr + qi::warp_sum(p);
#pragma unroll
        for (int i = 0; i < kAccPerLane; ++i) acc[i] *= corr;
        const int count = min(32, pos - base + 1);
        for (int jj = 0; jj < count; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int key = base + jj;
            const int page = table[key / page_size];
            if (page < 0 || page >= num_pages) continue;
            const T* vrow = cache + ((size_t)page * page_size + (key % page_size)) * (size_t)W;
#pragma unroll
            for (int i = 0; i < kAccPerLane; ++i) {
                const int idx = lane + 32 * i;
                if (idx < R) acc[i] = fmaf(pj, qi::to_f32<T>(vrow[idx]), acc[i]);
            }
        }
        m = m_new;
    }
    if (bad_page && status) atomicOr(status, qi::kStatusBadPage);

    if (lane == 0) {
        part_m[warp] = m;
        part_l[warp] = l;
    }
#pragma unroll
    for (int i = 0; i < kAccPerLane; ++i) {
        const int idx = lane + 32 * i;
        if (idx < R) part_acc[warp * R + idx] = acc[i];
    }
    __syncthreads();

    const float sk = sink ? sink[h] : -INFINITY;
    float gm = sk;
    for (int w = 0; w < kWarps; ++w) gm = fmaxf(gm, part_m[w]);
    float gl = sink ? expf(sk - gm) : 0.f;      // the sink's place in the denominator
    float wscale[kWarps];
    for (int w = 0; w < kWarps; ++w) {
        wscale[w] = (part_m[w] == -INFINITY) ? 0.f : expf(part_m[w] - gm);
        gl += part_l[w] * wscale[w];
    }
    T* orow = out + ((size_t)t * H + h) * R;
    for (int i = threadIdx.x; i < R; i += blockDim.x) {
        float o = 0.f;
        for (int w = 0; w < kWarps; ++w) o += part_acc[w * R + i] * wscale[w];
        orow[i] = qi::from_f32<T>(gl > 0.f ? o / gl : 0.f);
    }
}

}  // namespace

// proj [n, ldp] in `proj_dtype`: H heads of (d + r) from column 0, and from column kv_off (kv_off < 0: absent)
// the latent projection of R + r. q_out [n, H, R + r] in `dtype`: columns R .. R + r of every head are written.
// cache [num_pages, page_size, R + r] in `dtype`. gain float32 [R]; inv_freq float32 [rot_dims / 2].
extern "C" int qi_latent_prepare(const void* proj, int proj_dtype, long long ldp, int kv_off, void* q_out, int dtype,
                                 const float* gain, float eps, const float* inv_freq, int rot_dims,
                                 const int* positions, const int* token_req, const int* block_table, int max_blocks,
                                 int page_size, int num_pages, void* cache, int n_tokens, int H, int d, int r, int R,
                                 int half_split, float magnitude, int* status, cudaStream_t stream) {
    QI_REQUIRE(n_tokens >= 0 && H > 0 && d > 0 && r >= 0 && R > 0, "latent_prepare: bad sizes");
    QI_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= r, "latent_prepare: %d rotated coordinates do not fit a part of %d", rot_dims, r);
    QI_REQUIRE(rot_dims == 0 || inv_freq, "latent_prepare: the rotation's frequencies are missing");
    QI_REQUIRE(ldp >= (long long)H * (d + r) && (kv_off < 0 || ldp >= kv_off + R + r), "latent_prepare: the projection's rows are too short");
    if (kv_off >= 0) {
        QI_REQUIRE(cache && gain && block_table && page_size > 0 && max_blocks > 0 && num_pages > 0, "latent_prepare: the cache or the gain is missing");
        QI_REQUIRE(eps > 0.f, "latent_prepare: eps must be positive");
    }
    if (n_tokens == 0) return 0;
    const size_t smem = sizeof(float) * (rot_dims + 32);
    QI_DISPATCH_DTYPE(proj_dtype, TP, {
        QI_DISPATCH_DTYPE(dtype, T, {
            qi::launch(latent_prepare_kernel<TP, T>, dim3(n_tokens), dim3(128), smem, stream, (const TP*)proj, ldp, kv_off, (T*)q_out, gain,
                       eps, inv_freq, rot_dims, positions, token_req, block_table, max_blocks, page_size, num_pages, (T*)cache,
                       H, d, r, R, half_split, magnitude, status);
        });
    });
    return qi::check_launch("latent_prepare");
}

// q [n, H, W], out [n, H, R], cache [num_pages, page_size, W], all in `dtype`; sink float32 [H] or null.
extern "C" int qi_latent_attention_generic(const void* q, void* out, int dtype, const void* cache, const float* sink,
                                           const int* block_table, int max_blocks, int page_size, int num_pages,
                                           const int* positions, const int* token_req, int n_tokens, int H, int W,
                                           int R, float scale, int window, int* status, cudaStream_t stream) {
    QI_REQUIRE(n_tokens >= 0 && H > 0 && R > 0 && W >= R, "latent_attention: bad sizes");
    QI_REQUIRE(R <= kMaxR, "latent_attention: a latent of %d is above the limit %d of this kernel", R, kMaxR);
    QI_REQUIRE(page_size > 0 && max_blocks > 0 && num_pages > 0, "latent_attention: bad page geometry");
    QI_REQUIRE(window >= 0, "latent_attention: window must be >= 0 (0 = all keys)");
    QI_REQUIRE(H <= 65535, "latent_attention: too many heads for one launch");
    if (n_tokens == 0) return 0;
    const size_t smem = sizeof(float) * ((size_t)W + kWarps * R + 2 * kWarps);
    QI_REQUIRE(smem <= 48 * 1024, "latent_attention: rows of %d are too wide for this kernel", W);
    for (int t0 = 0; t0 < n_tokens; t0 += 65535) {
        const int nt = n_tokens - t0 < 65535 ? n_tokens - t0 : 65535;
        QI_DISPATCH_DTYPE(dtype, T, {
            qi::launch(latent_attention_generic_kernel<T>, dim3(H, nt), dim3(kWarps * 32), smem, stream,
                       (const T*)q + (size_t)t0 * H * W, (T*)out + (size_t)t0 * H * R, (const T*)cache, sink, block_table, max_blocks,
                       page_size, num_pages, positions + t0, token_req + t0, H, W, R, scale, window, status);
        });
    }
    return qi::check_launch("latent_attention_generic");
}

// bfloat16 attention on the tensor cores (mma.sync m16n8k16, 32-bit scores, softmax and accumulation) for
// mixers whose keys and values have sizes of their own (any multiples of 8 up to 128 each), whose
// visibility may be bounded by a chunk and a window besides causality, and whose result may pass an
// output gate:
//
//     s_ij = cap((q_i . k_j) * scale)    for lo(i) <= j <= i,   lo(i) = max(start of i's chunk, i - window + 1, 0)
//     out_i = (sum_j softmax(s_i)_j v_j) * sigmoid(gate_i) * out_scale      cap(s) = c tanh(s / c), or s without a cap
//
// One kernel serves prompts, portions and single decode tokens: a CTA of four warps takes up to 64
// consecutive query rows of ONE step entry and one query head (the tiles are found on the device from
// q_start, so the launch can sit in a CUDA graph), walks the keys its rows can see in tiles of 64 that
// start at multiples of 64 of the ABSOLUTE position (so a row's sums do not depend on where a prompt
// was cut), with the softmax evaluated online; the next tile is requested with cp.async into a second buffer
// while the current one is multiplied. Keys before the first visible one are zero-filled and
// never looked up: their pages may have gone back to the pool. Head sizes are padded with zeros to the
// next of 32, 64, 96, 128 in shared memory.
#include "common.cuh"

#include <math.h>

namespace {

constexpr int kQT = 64, kKT = 64, kThreads = 128, kPad = 8;

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Copies `rows` rows of `width` bf16 (width a multiple of 8) into a shared tile with row stride `stride`
// elements, zero beyond `width` up to `padded` and for rows the predicate refuses.
template <typename RowPtr>
__device__ __forceinline__ void fill_tile(qi::bf16* dst, int stride, int rows, int width, int padded, RowPtr row_ptr) {
    const int chunks = padded / 8;
    for (int idx = threadIdx.x; idx < rows * chunks; idx += kThreads) {
        const int r = idx / chunks, c = idx % chunks;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (c * 8 < width) {
            const qi::bf16* src = row_ptr(r);
            if (src) v = *reinterpret_cast<const uint4*>(src + c * 8);
        }
        *reinterpret_cast<uint4*>(dst + (size_t)r * stride + c * 8) = v;
    }
}

// The same with cp.async (16 bytes a request; a refused row or a padding column is zero-filled by a request of
// zero source bytes), for tiles that land while the tile before them is multiplied.
template <typename RowPtr>
__device__ __forceinline__ void fill_tile_async(qi::bf16* dst, int stride, int rows, int width, int padded, const qi::bf16* any, RowPtr row_ptr) {
    // two threads a row (64 rows, 128 threads): the row's page is looked up once, its 16-byte pieces are dealt out in turn
    static_assert(kThreads == 2 * kKT, "two threads a row");
    const int r = threadIdx.x >> 1;
    if (r >= rows) return;
    const qi::bf16* src = row_ptr(r);
    const uint32_t d0 = (uint32_t)__cvta_generic_to_shared(dst + (size_t)r * stride);
    for (int c = threadIdx.x & 1; c * 8 < padded; c += 2) {
        const bool real = src && c * 8 < width;
        const int bytes = real ? 16 : 0;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d0 + c * 16), "l"(real ? (const void*)(src + c * 8) : (const void*)any), "r"(bytes) : "memory");
    }
}

template <int DK, int DV>
__global__ void __launch_bounds__(kThreads)
gated_attention_mma_kernel(const qi::bf16* __restrict__ q, qi::bf16* __restrict__ out, const qi::bf16* __restrict__ k_pages,
                           const qi::bf16* __restrict__ v_pages, const int* __restrict__ block_table, int max_blocks,
                           int page_size, int num_pages, const int* __restrict__ q_start, const int* __restrict__ start_pos,
                           int n_entries, int nq, int nkv, int d, int dv, float scale_log2e, float softcap, float out_scale,
                           int window, int chunk, const qi::bf16* __restrict__ gate, long long ldg, const float* __restrict__ sink,
                           int n_ranges, float* __restrict__ ws_o, float* __restrict__ ws_ml, int* __restrict__ status) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    constexpr int SK = DK + kPad, SV = DV + kPad;
    qi::bf16* Qs = reinterpret_cast<qi::bf16*>(smem_raw);       // [kQT][SK]
    qi::bf16* Kbuf = Qs + kQT * SK;                              // 2 x [kKT][SK]
    qi::bf16* Vbuf = Kbuf + 2 * kKT * SK;                        // 2 x [kKT][SV]

    qi::pdl_wait();
    // which tile of which entry this CTA takes
    int e = -1, row0 = 0, rows = 0, pos0 = 0;
    {
        int acc = 0;
        for (int i = 0; i < n_entries; ++i) {
            const int a = q_start[i], len = q_start[i + 1] - a;
            const int nt = (len + kQT - 1) / kQT;
            if ((int)blockIdx.x < acc + nt) {
                const int off = ((int)blockIdx.x - acc) * kQT;
                e = i; row0 = a + off; rows = min(kQT, len - off); pos0 = start_pos[i] + off;
                break;
            }
            acc += nt;
        }
    }
    if (e < 0) return;
    const int h = blockIdx.y, hk = h / (nq / nkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* table = block_table + (size_t)e * max_blocks;

    auto row_lo = [&](int p) {
        int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
        if (chunk > 0) lo = max(lo, p / chunk * chunk);
        return lo;
    };
    const int lo_min = row_lo(pos0);              // lo is monotone in the position
    const int hi = pos0 + rows - 1;               // the last row's own position

    fill_tile(Qs, SK, kQT, d, DK, [&](int r) -> const qi::bf16* {
        return r < rows ? q + ((size_t)(row0 + r) * nq + h) * d : nullptr;
    });
    __syncthreads();
    // this warp's 16 rows of Q as A fragments
    uint32_t qa[DK / 16][4];
    {
        const int r = warp * 16 + (lane >> 2), c = (lane & 3) * 2;
#pragma unroll
        for (int kk = 0; kk < DK / 16; ++kk) {
            qa[kk][0] = *reinterpret_cast<const uint32_t*>(Qs + (size_t)r * SK + kk * 16 + c);
            qa[kk][1] = *reinterpret_cast<const uint32_t*>(Qs + (size_t)(r + 8) * SK + kk * 16 + c);
            qa[kk][2] = *reinterpret_cast<const uint32_t*>(Qs + (size_t)r * SK + kk * 16 + 8 + c);
            qa[kk][3] = *reinterpret_cast<const uint32_t*>(Qs + (size_t)(r + 8) * SK + kk * 16 + 8 + c);
        }
    }
    const int rA = warp * 16 + (lane >> 2), rB = rA + 8;          // this thread's two rows of the tile
    const int pA = pos0 + rA, pB = pos0 + rB;
    const int loA = row_lo(pA), loB = row_lo(pB);
    float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;
    float o[DV / 8][4];
#pragma unroll
    for (int n = 0; n < DV / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

    bool bad_page = false;
    auto request_tile = [&](int t0, int buf) {
        auto page_row = [&](int r, const qi::bf16* pages, int width) -> const qi::bf16* {
            const int key = t0 + r;
            if (key < lo_min || key > hi) return nullptr;
            const int page = table[key / page_size];
            if (page < 0 || page >= num_pages) { bad_page = true; return nullptr; }
            return pages + (((size_t)page * nkv + hk) * page_size + (key % page_size)) * (size_t)width;
        };
        fill_tile_async(Kbuf + (size_t)buf * kKT * SK, SK, kKT, d, DK, k_pages, [&](int r) { return page_row(r, k_pages, d); });
        fill_tile_async(Vbuf + (size_t)buf * kKT * SV, SV, kKT, dv, DV, k_pages, [&](int r) { return page_row(r, v_pages, dv); });
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    int t_first = lo_min / kKT * kKT, t_last = hi;
    if (n_ranges > 1) {
        // the tile's key tiles in n_ranges equal parts, one a CTA along grid.z; a merge kernel adds the parts
        const int per = ((hi - t_first) / kKT + n_ranges) / n_ranges;
        t_first += (int)blockIdx.z * per * kKT;
        t_last = min(hi, t_first + per * kKT - 1);
    }
    int buf = 0;
    if (t_first <= t_last) request_tile(t_first, 0);
    for (int t0 = t_first; t0 <= t_last; t0 += kKT, buf ^= 1) {
        if (t0 + kKT <= t_last) {        // the next tile lands while this one is multiplied
            request_tile(t0 + kKT, buf ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const qi::bf16* Ks = Kbuf + (size_t)buf * kKT * SK;
        const qi::bf16* Vs = Vbuf + (size_t)buf * kKT * SV;

        float s[kKT / 8][4];
#pragma unroll
        for (int n = 0; n < kKT / 8; ++n) {
            s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
            const qi::bf16* kr = Ks + (size_t)(n * 8 + (lane >> 2)) * SK + (lane & 3) * 2;
#pragma unroll
            for (int kk = 0; kk < DK / 16; ++kk)
                mma_bf16(s[n], qa[kk], *reinterpret_cast<const uint32_t*>(kr + kk * 16), *reinterpret_cast<const uint32_t*>(kr + kk * 16 + 8));
        }
        // soft cap: c tanh(s scale / c), then into the base-2 exponent like the plain scale
        if (softcap > 0.f) {
            const float a = scale_log2e * (0.6931471805599453f / softcap), b = softcap * 1.4426950408889634f / scale_log2e;
#pragma unroll
            for (int n = 0; n < kKT / 8; ++n) {
#pragma unroll
                for (int j = 0; j < 4; ++j) s[n][j] = b * tanhf(s[n][j] * a);
            }
        }
        // mask, scale (into the base-2 exponent), row maxima
        float tmA = -INFINITY, tmB = -INFINITY;
#pragma unroll
        for (int n = 0; n < kKT / 8; ++n) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int key = t0 + n * 8 + (lane & 3) * 2 + j;
                s[n][j] = (key >= loA && key <= pA && rA < rows) ? s[n][j] * scale_log2e : -INFINITY;
                s[n][2 + j] = (key >= loB && key <= pB && rB < rows) ? s[n][2 + j] * scale_log2e : -INFINITY;
                tmA = fmaxf(tmA, s[n][j]);
                tmB = fmaxf(tmB, s[n][2 + j]);
            }
        }
        tmA = fmaxf(tmA, __shfl_xor_sync(0xffffffffu, tmA, 1)); tmA = fmaxf(tmA, __shfl_xor_sync(0xffffffffu, tmA, 2));
        tmB = fmaxf(tmB, __shfl_xor_sync(0xffffffffu, tmB, 1)); tmB = fmaxf(tmB, __shfl_xor_sync(0xffffffffu, tmB, 2));
        const float nmA = fmaxf(mA, tmA), nmB = fmaxf(mB, tmB);
        const float baseA = nmA == -INFINITY ? 0.f : nmA, baseB = nmB == -INFINITY ? 0.f : nmB;
        const float cA = exp2f(mA - baseA), cB = exp2f(mB - baseB);       // m = -inf gives 0
        mA = nmA; mB = nmB;
        float sumA = 0.f, sumB = 0.f;
#pragma unroll
        for (int n = 0; n < kKT / 8; ++n) {
            s[n][0] = exp2f(s[n][0] - baseA); s[n][1] = exp2f(s[n][1] - baseA);
            s[n][2] = exp2f(s[n][2] - baseB); s[n][3] = exp2f(s[n][3] - baseB);
            sumA += s[n][0] + s[n][1];
            sumB += s[n][2] + s[n][3];
        }
        lA = lA * cA + sumA;      // the four lanes of a row keep partial sums; they meet at the end
        lB = lB * cB + sumB;
#pragma unroll
        for (int n = 0; n < DV / 8; ++n) { o[n][0] *= cA; o[n][1] *= cA; o[n][2] *= cB; o[n][3] *= cB; }
        // O += P V
#pragma unroll
        for (int kk = 0; kk < kKT / 16; ++kk) {
            uint32_t pa[4];
            pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int n2 = 0; n2 < DV / 16; ++n2) {
                uint32_t b0, b1, b2, b3;
                const qi::bf16* vr = Vs + (size_t)(kk * 16 + (lane & 15)) * SV + n2 * 16 + (lane >> 4) * 8;
                const uint32_t addr = (uint32_t)__cvta_generic_to_shared(vr);
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(addr));
                mma_bf16(o[2 * n2], pa, b0, b1);
                mma_bf16(o[2 * n2 + 1], pa, b2, b3);
            }
        }
        __syncthreads();                 // every warp is done with this buffer before the tile after next is requested into it
    }
    if (bad_page && status) atomicOr(status, qi::kStatusBadPage);
    lA += __shfl_xor_sync(0xffffffffu, lA, 1); lA += __shfl_xor_sync(0xffffffffu, lA, 2);
    lB += __shfl_xor_sync(0xffffffffu, lB, 1); lB += __shfl_xor_sync(0xffffffffu, lB, 2);
    if (n_ranges > 1) {       // this part's reference, sum and accumulator as they are; the merge kernel finishes the rows
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = half ? rB : rA;
            if (r >= rows) continue;
            const size_t slot = ((size_t)(row0 + r) * nq + h) * n_ranges + blockIdx.z;
            if ((lane & 3) == 0) {
                ws_ml[slot * 2] = half ? mB : mA;
                ws_ml[slot * 2 + 1] = half ? lB : lA;
            }
#pragma unroll
            for (int n = 0; n < DV / 8; ++n) {
                const int col = n * 8 + (lane & 3) * 2;
                if (col < dv) {
                    ws_o[slot * dv + col] = o[n][2 * half];
                    ws_o[slot * dv + col + 1] = o[n][2 * half + 1];
                }
            }
        }
        return;
    }
    if (sink) {       // one more term in the denominator, exp(sink_h), with no key and no value (m is a base-2 exponent)
        const float sb = sink[h] * 1.4426950408889634f;
        if (mA != -INFINITY) lA += exp2f(sb - mA);
        if (mB != -INFINITY) lB += exp2f(sb - mB);
    }
    const float iA = lA > 0.f ? 1.0f / lA : 0.f, iB = lB > 0.f ? 1.0f / lB : 0.f;   // out_scale joins below, after the gate
#pragma unroll
    for (int n = 0; n < DV / 8; ++n) {
        const int col = n * 8 + (lane & 3) * 2;
        if (col >= dv) continue;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = half ? rB : rA;
            if (r >= rows) continue;
            float v0 = o[n][2 * half] * (half ? iB : iA), v1 = o[n][2 * half + 1] * (half ? iB : iA);
            const size_t t = (size_t)(row0 + r);
            if (gate) {
                const qi::bf16* g = gate + t * ldg + (size_t)h * dv + col;
                v0 = v0 / (1.0f + expf(-__bfloat162float(g[0])));
                v1 = v1 / (1.0f + expf(-__bfloat162float(g[1])));
            }
            *reinterpret_cast<__nv_bfloat162*>(out + (t * nq + h) * dv + col) = __floats2bfloat162_rn(v0 * out_scale, v1 * out_scale);
        }
    }
}

// out[t, h, :] = sum_s o_s 2^(m_s - M) / (sum_s l_s 2^(m_s - M) + 2^(sink_h log2 e - M)), then the gate and the factor:
// the parts of a row that the key ranges left, added in range order.
__global__ void gated_attention_merge_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_ml, qi::bf16* __restrict__ out,
                                             int nq, int dv, int n_ranges, const qi::bf16* __restrict__ gate, long long ldg,
                                             const float* __restrict__ sink, float out_scale) {
    qi::pdl_wait();
    const int h = blockIdx.x;
    const size_t t = blockIdx.y;
    const size_t base = (t * nq + h) * n_ranges;
    float M = -INFINITY;
    for (int s = 0; s < n_ranges; ++s) M = fmaxf(M, ws_ml[(base + s) * 2]);
    const float sink_term = (sink && M != -INFINITY) ? exp2f(sink[h] * 1.4426950408889634f - M) : 0.f;
    for (int col = threadIdx.x; col < dv; col += blockDim.x) {
        float L = sink_term, O = 0.f;
        for (int s = 0; s < n_ranges; ++s) {
            const float ms = ws_ml[(base + s) * 2];
            if (ms == -INFINITY) continue;          // a part without keys
            const float f = exp2f(ms - M);
            L += ws_ml[(base + s) * 2 + 1] * f;
            O += ws_o[(base + s) * dv + col] * f;
        }
        float v = L > 0.f ? O / L : 0.f;
        if (gate) v = v / (1.0f + expf(-__bfloat162float(gate[t * (size_t)ldg + (size_t)h * dv + col])));
        out[(t * nq + h) * dv + col] = __float2bfloat16_rn(v * out_scale);
    }
}

int padded(int v) { return v <= 32 ? 32 : v <= 64 ? 64 : v <= 96 ? 96 : 128; }

template <int DK, int DV>
int launch_one(dim3 grid, cudaStream_t stream, const void* q, void* out, const void* k_pages, const void* v_pages,
               const int* block_table, int max_blocks, int page_size, int num_pages, const int* q_start, const int* start_pos,
               int n_entries, int nq, int nkv, int d, int dv, float scale_log2e, float softcap, float out_scale, int window, int chunk,
               const void* gate, long long ldg, const float* sink, int n_ranges, float* ws_o, float* ws_ml, int n_tokens, int* status) {
    const size_t smem = sizeof(qi::bf16) * ((size_t)(kQT + 2 * kKT) * (DK + kPad) + (size_t)2 * kKT * (DV + kPad));
    static bool raised = false;
    if (!raised && smem > 48 * 1024) {
        cudaFuncSetAttribute(gated_attention_mma_kernel<DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        raised = true;
    }
    qi::launch(gated_attention_mma_kernel<DK, DV>, grid, dim3(kThreads), smem, stream, (const qi::bf16*)q, (qi::bf16*)out,
               (const qi::bf16*)k_pages, (const qi::bf16*)v_pages, block_table, max_blocks, page_size, num_pages, q_start, start_pos,
               n_entries, nq, nkv, d, dv, scale_log2e, softcap, out_scale, window, chunk, (const qi::bf16*)gate, ldg, sink, n_ranges, ws_o, ws_ml, status);
    if (n_ranges > 1) {
        if (int rc = qi::check_launch("gated_attention_mma")) return rc;
        qi::launch(gated_attention_merge_kernel, dim3(nq, n_tokens), dim3(128), 0, stream, (const float*)ws_o, (const float*)ws_ml,
                   (qi::bf16*)out, nq, dv, n_ranges, (const qi::bf16*)gate, ldg, sink, out_scale);
        return qi::check_launch("gated_attention_merge");
    }
    return qi::check_launch("gated_attention_mma");
}

}  // namespace

extern "C" int qi_gated_attention_mma_supported(int nq, int nkv, int d, int dv) {
    return nq > 0 && nkv > 0 && nq % nkv == 0 && d > 0 && dv > 0 && d % 8 == 0 && dv % 8 == 0 && d <= 128 && dv <= 128;
}

// q [n, nq d], out [n, nq dv], pages [num_pages, nkv, page_size, d | dv], all bfloat16; q_start [entries + 1],
// start_pos [entries]; gate (may be null) row t, head h, element i at gate[t * ldg + h * dv + i] (ldg and dv even);
// softcap c > 0: a score s becomes c tanh(s / c) before the softmax; out_scale multiplies the result. sink (may be null):
// float32 [nq]; the softmax's denominator of head h holds exp(sink[h]) once more.
// n_ranges > 1 (steps of single tokens over long contexts): every query tile's keys are cut into that many ranges over
// separate CTAs and a second kernel adds the parts; `workspace` must then hold n_tokens * nq * n_ranges * (dv + 2) floats.
extern "C" int qi_gated_attention_mma_ranges(const void* q, void* out, const void* k_pages, const void* v_pages, const int* block_table,
                                      int max_blocks, int page_size, int num_pages, const int* q_start, const int* start_pos,
                                      int n_entries, int n_tokens, int nq, int nkv, int d, int dv, float scale, float softcap,
                                      float out_scale, int window, int chunk, const void* gate, long long ldg, const float* sink,
                                      int n_ranges, float* workspace, int* status, cudaStream_t stream) {
    QI_REQUIRE(n_ranges >= 1 && n_ranges <= 64 && (n_ranges == 1 || (workspace && n_tokens <= 65535)), "gated_attention_mma: key ranges need a workspace (1 to 64 ranges, at most 65535 tokens)");
    QI_REQUIRE(qi_gated_attention_mma_supported(nq, nkv, d, dv), "gated_attention_mma: heads %d/%d of %d/%d are not covered", nq, nkv, d, dv);
    QI_REQUIRE(n_entries >= 0 && n_tokens >= 0 && page_size > 0 && max_blocks > 0 && num_pages > 0, "gated_attention_mma: bad sizes");
    QI_REQUIRE(window >= 0 && chunk >= 0, "gated_attention_mma: window and chunk must be >= 0 (0 = none)");
    QI_REQUIRE(softcap >= 0.f && scale > 0.f, "gated_attention_mma: the soft cap must be >= 0 (0 = none) and the scale positive");
    QI_REQUIRE(!gate || (ldg >= (long long)nq * dv && ldg % 2 == 0), "gated_attention_mma: the gate's rows are too short or odd");
    QI_REQUIRE(nq <= 65535, "gated_attention_mma: too many heads");
    if (n_tokens == 0 || n_entries == 0) return 0;
    const dim3 grid(n_tokens / kQT + n_entries, nq, n_ranges);
    float* ws_o = workspace;
    float* ws_ml = workspace ? workspace + (size_t)n_tokens * nq * n_ranges * dv : nullptr;
    const float sl = scale * 1.4426950408889634f;
#define QI_GA(DKP, DVP)                                                                                                      \
    return launch_one<DKP, DVP>(grid, stream, q, out, k_pages, v_pages, block_table, max_blocks, page_size, num_pages, q_start, \
                                start_pos, n_entries, nq, nkv, d, dv, sl, softcap, out_scale, window, chunk, gate, ldg, sink, n_ranges, ws_o, ws_ml, n_tokens, status)
#define QI_GA_ROW(DKP)                                   \
    switch (padded(dv)) {                                \
        case 32: QI_GA(DKP, 32);                         \
        case 64: QI_GA(DKP, 64);                         \
        case 96: QI_GA(DKP, 96);                         \
        default: QI_GA(DKP, 128);                        \
    }
    switch (padded(d)) {
        case 32: QI_GA_ROW(32);
        case 64: QI_GA_ROW(64);
        case 96: QI_GA_ROW(96);
        default: QI_GA_ROW(128);
    }
#undef QI_GA_ROW
#undef QI_GA
    return 0;
}

extern "C" int qi_gated_attention_mma_sink(const void* q, void* out, const void* k_pages, const void* v_pages, const int* block_table,
                                      int max_blocks, int page_size, int num_pages, const int* q_start, const int* start_pos,
                                      int n_entries, int n_tokens, int nq, int nkv, int d, int dv, float scale, float softcap,
                                      float out_scale, int window, int chunk, const void* gate, long long ldg, const float* sink,
                                      int* status, cudaStream_t stream);

extern "C" int qi_gated_attention_mma(const void* q, void* out, const void* k_pages, const void* v_pages, const int* block_table,
                                      int max_blocks, int page_size, int num_pages, const int* q_start, const int* start_pos,
                                      int n_entries, int n_tokens, int nq, int nkv, int d, int dv, float scale, float softcap,
                                      float out_scale, int window, int chunk, const void* gate, long long ldg, int* status, cudaStream_t stream) {
    return qi_gated_attention_mma_sink(q, out, k_pages, v_pages, block_table, max_blocks, page_size, num_pages, q_start, start_pos,
                                       n_entries, n_tokens, nq, nkv, d, dv, scale, softcap, out_scale, window, chunk, gate, ldg, nullptr,
                                       status, stream);
}

extern "C" int qi_gated_attention_mma_sink(const void* q, void* out, const void* k_pages, const void* v_pages, const int* block_table,
                                      int max_blocks, int page_size, int num_pages, const int* q_start, const int* start_pos,
                                      int n_entries, int n_tokens, int nq, int nkv, int d, int dv, float scale, float softcap,
                                      float out_scale, int window, int chunk, const void* gate, long long ldg, const float* sink,
                                      int* status, cudaStream_t stream) {
    return qi_gated_attention_mma_ranges(q, out, k_pages, v_pages, block_table, max_blocks, page_size, num_pages, q_start, start_pos,
                                         n_entries, n_tokens, nq, nkv, d, dv, scale, softcap, out_scale, window, chunk, gate, ldg, sink, 1,
                                         nullptr, status, stream);
}

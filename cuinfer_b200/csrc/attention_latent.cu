// Attention over a cache of latents: every token keeps ONE row [c (rk values) | k_rot (dr values)] shared by all heads,
// instead of keys and values per head.  c is the RMS-normed down-projection from which a head's keys and values
// would be up-projected (k_h = Uk_h c, v_h = Uv_h c); k_rot is a rotary-encoded key part common to the heads.
// With the up-projections moved to the query and output side,
//     score_h(i, j) = scale * ( (Uk_h^T q_h(i)) . c(j) + rot(q_rot_h(i)) . k_rot(j) ),
//     out_h(i)      = Uv_h * sum_j w_h(i, j) c(j),
// the kernel is multi-query attention whose keys are the cached rows (rk + dr wide) and whose values are the first rk
// columns of the same rows.  The softmax may carry a sink: a per-head number whose exponential joins the denominator,
// without key or value.
//
// Two kernels:
//  * latent_prep: per token, RMS norm of the query latent (written out for the query up-projection), RMS norm of the
//    key/value latent and rotary encoding of the shared key part, both written to the token's cache slot.  Pairs are
//    interleaved, (2i, 2i+1), over the first `rot_dims` of the dr values; the angle is position * freq[i] in 32 bits
//    with the full-range sine and cosine, both multiplied by `rot_gain` (1: a pure rotation).  Without a query latent
//    (no output for it) only the cache row is written.
//  * latent_attention_generic: a warp per (query token, head), any sizes up to rk = 1024, 32-bit throughout with
//    the exact exponential; the query's rotary part is encoded as it is loaded.  This is the 32-bit path and the
//    fallback of the tensor-core kernels.
//
// Cache layout of one layer run: [page][slot in page][rk + dr].
#include "common.cuh"

namespace cib {

template <typename T>
__global__ void latent_prep_kernel(const T* __restrict__ proj, int stride, int q_off, int rq, int kv_off, int rk, int dr,
                                   AnyVec q_gain, AnyVec kv_gain, float eps, const int* __restrict__ positions,
                                   const float* __restrict__ freq, int rot_dims, float rot_gain,
                                   const int* __restrict__ slot_mapping, T* __restrict__ cache, long long num_slots,
                                   T* __restrict__ cq_out, int cq_stride) {
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const T* row = proj + (size_t)t * stride;
    // query latent
    if (cq_out) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < rq; i += blockDim.x) {
            const float v = to_f32(row[q_off + i]);
            ss += v * v;
        }
        const float f = 1.f / sqrtf(block_sum(ss, scratch) / (float)rq + eps);
        for (int i = threadIdx.x; i < rq; i += blockDim.x)
            cq_out[(size_t)t * cq_stride + i] = from_f32<T>(to_f32(row[q_off + i]) * f * q_gain[i]);
    }
    // key/value latent and the shared rotary key part, to the token's slot
    const long long slot = slot_mapping ? slot_mapping[t] : -1;
    if (!cache || slot < 0 || slot >= num_slots) return;          // uniform over the block
    T* dst = cache + (size_t)slot * (rk + dr);
    float ss = 0.f;
    for (int i = threadIdx.x; i < rk; i += blockDim.x) {
        const float v = to_f32(row[kv_off + i]);
        ss += v * v;
    }
    const float f = 1.f / sqrtf(block_sum(ss, scratch) / (float)rk + eps);
    for (int i = threadIdx.x; i < rk; i += blockDim.x) dst[i] = from_f32<T>(to_f32(row[kv_off + i]) * f * kv_gain[i]);
    const float pos = (float)positions[t];
    const T* kr = row + kv_off + rk;
    for (int i = threadIdx.x; i < dr / 2; i += blockDim.x) {
        const float u = to_f32(kr[2 * i]), v = to_f32(kr[2 * i + 1]);
        if (2 * i + 1 < rot_dims) {
            float s, c;
            sincosf(pos * freq[i], &s, &c);
            s *= rot_gain;
            c *= rot_gain;
            dst[rk + 2 * i] = from_f32<T>(u * c - v * s);
            dst[rk + 2 * i + 1] = from_f32<T>(v * c + u * s);
        } else {
            dst[rk + 2 * i] = kr[2 * i];
            dst[rk + 2 * i + 1] = kr[2 * i + 1];
        }
    }
    if ((dr & 1) && threadIdx.x == 0) dst[rk + dr - 1] = kr[dr - 1];
}

constexpr int kLatentWarps = 4;

// q_abs: [T][H][rk] 32-bit or T (`TQ`), rows `qa_stride` apart, heads rk apart.
// q:     [T][H][dn + dr] packed rows, of which the last dr of a head are its rotary part (not yet encoded).
template <typename T, typename TQ, int ACC>
__global__ void latent_attention_generic_kernel(
    const TQ* __restrict__ q_abs, int qa_stride, const T* __restrict__ q, int q_stride, int dn, T* __restrict__ out,
    int out_stride, const T* __restrict__ cache, int num_pages, int page_size, const int* __restrict__ block_table,
    int table_stride, const int* __restrict__ query_start_loc, const int* __restrict__ seq_lens,
    const int* __restrict__ token_request, const int* __restrict__ positions, const float* __restrict__ freq, int rot_dims,
    float rot_gain, AnyVec sinks, int has_sink, int H, int rk, int dr, float scale, int window) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int head = blockIdx.y * kLatentWarps + warp;
    if (head >= H) return;
    const int D = rk + dr;
    float* qs = smem + warp * D;

    const int r = token_request[t];
    const int q0 = query_start_loc[r];
    const int n = query_start_loc[r + 1] - q0;
    const int pos = seq_lens[r] - n + (t - q0);
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int* table = block_table + (size_t)r * table_stride;

    const TQ* qa = q_abs + (size_t)t * qa_stride + (size_t)head * rk;
    for (int i = lane; i < rk; i += 32) qs[i] = to_f32(qa[i]) * scale;
    const T* qr = q + (size_t)t * q_stride + (size_t)head * (dn + dr) + dn;
    const float fpos = (float)positions[t];
    for (int i = lane; i < dr / 2; i += 32) {
        const float u = to_f32(qr[2 * i]), v = to_f32(qr[2 * i + 1]);
        if (2 * i + 1 < rot_dims) {
            float s, c;
            sincosf(fpos * freq[i], &s, &c);
            s *= rot_gain;
            c *= rot_gain;
            qs[rk + 2 * i] = (u * c - v * s) * scale;
            qs[rk + 2 * i + 1] = (v * c + u * s) * scale;
        } else {
            qs[rk + 2 * i] = u * scale;
            qs[rk + 2 * i + 1] = v * scale;
        }
    }
    if ((dr & 1) && lane == 0) qs[D - 1] = to_f32(qr[dr - 1]) * scale;
    __syncwarp();

    float acc[ACC];
#pragma unroll
    for (int k = 0; k < ACC; ++k) acc[k] = 0.f;
    // the sink is a score without key or value: it starts the running maximum and counts once in the sum
    float m = has_sink ? sinks[head] : -INFINITY;
    float l = has_sink ? 1.f : 0.f;

    for (int c0 = lo; c0 <= pos; c0 += 32) {
        const int j = c0 + lane;
        int page = -1, off = 0;
        float s = -INFINITY;
        if (j <= pos) {
            page = table[j / page_size];
            off = j % page_size;
            if (page >= 0 && page < num_pages) {
                const T* kp = cache + ((size_t)page * page_size + off) * D;
                float dot = 0.f;
                for (int i = 0; i < D; ++i) dot = fmaf(qs[i], to_f32(kp[i]), dot);
                s = dot;
            } else {
                page = -1;
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;
        const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int k = 0; k < ACC; ++k) acc[k] *= corr;
        const int count = min(32, pos - c0 + 1);
        for (int jj = 0; jj < count; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int pg = __shfl_sync(0xffffffffu, page, jj);
            const int of = __shfl_sync(0xffffffffu, off, jj);
            if (pg < 0) continue;
            const T* vp = cache + ((size_t)pg * page_size + of) * D;
#pragma unroll
            for (int k = 0; k < ACC; ++k) {
                const int i = lane + 32 * k;
                if (i < rk) acc[k] = fmaf(pj, to_f32(vp[i]), acc[k]);
            }
        }
    }
    T* op = out + (size_t)t * out_stride + (size_t)head * rk;
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int k = 0; k < ACC; ++k) {
        const int i = lane + 32 * k;
        if (i < rk) op[i] = from_f32<T>(acc[k] * inv);
    }
}

}  // namespace cib

using namespace cib;

extern "C" int cib_latent_prep(const void* proj, int dtype, int stride, int q_off, int rq, int kv_off, int rk, int dr,
                               const void* q_gain, const void* kv_gain, int gain_dtype, float eps, const int* positions,
                               const float* freq, int rot_dims, float rot_gain, const int* slot_mapping, void* cache,
                               long long num_slots, void* cq_out, int cq_stride, int num_tokens, cudaStream_t stream) {
    CIB_REQUIRE(num_tokens >= 0 && rq >= 0 && rk > 0 && dr >= 0, "latent_prep: bad sizes T=%d rq=%d rk=%d dr=%d", num_tokens, rq, rk, dr);
    CIB_REQUIRE(rot_dims >= 0 && rot_dims <= dr && rot_dims % 2 == 0, "latent_prep: %d rotary dimensions in a part of %d", rot_dims, dr);
    CIB_REQUIRE(q_off >= 0 && kv_off >= 0 && q_off + rq <= stride && kv_off + rk + dr <= stride, "latent_prep: parts outside the rows");
    CIB_REQUIRE(rot_dims == 0 || freq != nullptr, "latent_prep: rotary dimensions without frequencies");
    if (num_tokens == 0) return 0;
    AnyVec qg{q_gain, gain_dtype == kBF16}, kg{kv_gain, gain_dtype == kBF16};
    if (dtype == kF32)
        latent_prep_kernel<float><<<num_tokens, 128, 0, stream>>>((const float*)proj, stride, q_off, rq, kv_off, rk, dr, qg, kg, eps, positions, freq, rot_dims, rot_gain, slot_mapping, (float*)cache, num_slots, (float*)cq_out, cq_stride);
    else if (dtype == kBF16)
        latent_prep_kernel<__nv_bfloat16><<<num_tokens, 128, 0, stream>>>((const __nv_bfloat16*)proj, stride, q_off, rq, kv_off, rk, dr, qg, kg, eps, positions, freq, rot_dims, rot_gain, slot_mapping, (__nv_bfloat16*)cache, num_slots, (__nv_bfloat16*)cq_out, cq_stride);
    else
        CIB_REQUIRE(false, "latent_prep: unsupported dtype %d", dtype);
    CIB_LAUNCH_CHECK("latent_prep");
    return 0;
}

template <typename T, typename TQ>
static void launch_latent_generic(int acc, dim3 grid, size_t smem, cudaStream_t stream, const void* q_abs, int qa_stride,
                                  const void* q, int q_stride, int dn, void* out, int out_stride, const void* cache,
                                  int num_pages, int page_size, const int* bt, int ts, const int* qsl, const int* sl,
                                  const int* tr, const int* positions, const float* freq, int rot_dims, float rot_gain,
                                  AnyVec sinks, int has_sink, int H, int rk, int dr, float scale, int window) {
#define CIB_LATENT_GO(A)                                                                                                  \
    latent_attention_generic_kernel<T, TQ, A><<<grid, kLatentWarps * 32, smem, stream>>>(                                  \
        (const TQ*)q_abs, qa_stride, (const T*)q, q_stride, dn, (T*)out, out_stride, (const T*)cache, num_pages, page_size, \
        bt, ts, qsl, sl, tr, positions, freq, rot_dims, rot_gain, sinks, has_sink, H, rk, dr, scale, window)
    if (acc <= 4) CIB_LATENT_GO(4);
    else if (acc <= 8) CIB_LATENT_GO(8);
    else if (acc <= 16) CIB_LATENT_GO(16);
    else CIB_LATENT_GO(32);
#undef CIB_LATENT_GO
}

extern "C" int cib_latent_attention_generic(const void* q_abs, int qa_dtype, int qa_stride, const void* q, int dtype,
                                            int q_stride, int dn, void* out, int out_stride, const void* cache,
                                            int num_pages, int page_size, const int* block_table, int table_stride,
                                            const int* query_start_loc, const int* seq_lens, const int* token_request,
                                            const int* positions, const float* freq, int rot_dims, float rot_gain,
                                            const void* sinks, int sink_dtype, int num_tokens, int H, int rk, int dr,
                                            float scale, int window, cudaStream_t stream) {
    CIB_REQUIRE(num_tokens >= 0 && H > 0 && rk > 0 && dr >= 0 && dn >= 0, "latent_attention: bad sizes T=%d H=%d rk=%d dr=%d", num_tokens, H, rk, dr);
    CIB_REQUIRE(rk <= 1024, "latent_attention: latent size %d exceeds 1024", rk);
    CIB_REQUIRE(page_size > 0 && num_pages > 0 && table_stride > 0, "latent_attention: bad cache geometry");
    CIB_REQUIRE(rot_dims >= 0 && rot_dims <= dr && rot_dims % 2 == 0 && (rot_dims == 0 || freq), "latent_attention: bad rotary part");
    CIB_REQUIRE(window >= 0, "latent_attention: window must be >= 0 (0 = all keys)");
    CIB_REQUIRE(qa_dtype == kF32 || qa_dtype == dtype, "latent_attention: absorbed queries must be 32-bit or of the rows' type");
    if (num_tokens == 0) return 0;
    dim3 grid(num_tokens, (H + kLatentWarps - 1) / kLatentWarps);
    const size_t smem = (size_t)kLatentWarps * (rk + dr) * sizeof(float);
    const int acc = (rk + 31) / 32;
    AnyVec sk{sinks, sink_dtype == kBF16};
    const int has_sink = sinks != nullptr;
    if (dtype == kF32)
        launch_latent_generic<float, float>(acc, grid, smem, stream, q_abs, qa_stride, q, q_stride, dn, out, out_stride, cache, num_pages, page_size, block_table, table_stride, query_start_loc, seq_lens, token_request, positions, freq, rot_dims, rot_gain, sk, has_sink, H, rk, dr, scale, window);
    else if (dtype == kBF16 && qa_dtype == kF32)
        launch_latent_generic<__nv_bfloat16, float>(acc, grid, smem, stream, q_abs, qa_stride, q, q_stride, dn, out, out_stride, cache, num_pages, page_size, block_table, table_stride, query_start_loc, seq_lens, token_request, positions, freq, rot_dims, rot_gain, sk, has_sink, H, rk, dr, scale, window);
    else if (dtype == kBF16)
        launch_latent_generic<__nv_bfloat16, __nv_bfloat16>(acc, grid, smem, stream, q_abs, qa_stride, q, q_stride, dn, out, out_stride, cache, num_pages, page_size, block_table, table_stride, query_start_loc, seq_lens, token_request, positions, freq, rot_dims, rot_gain, sk, has_sink, H, rk, dr, scale, window);
    else
        CIB_REQUIRE(false, "latent_attention: unsupported dtype %d", dtype);
    CIB_LAUNCH_CHECK("latent_attention_generic");
    return 0;
}

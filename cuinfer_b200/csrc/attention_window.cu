// Grouped-query attention whose keys and values have sizes of their own, with a capped score and a window that keeps
// the first tokens of a sequence visible: the step before the attention (biases, norm, rotation, query temperature, value
// mixing, cache write) and the plain all-sizes attention kernel (a warp per query token and head), which is the 32-bit
// path.  Every step is optional, so that one pair of kernels serves several kinds of attention layer.
//
// Per token and head, with the query q and key k of d values and the value v of dv values:
//   q, k, v += their biases (32-bit);
//   with `value_from_key` there is no v in the rows: v = k as it stands here, before norm and rotation;
//   rotation of the first `rot_dims` values by the angle pos * freq[i] (32-bit angle, full-range sine and cosine, both
//   multiplied by `rot_gain`), in neighbouring pairs (2i, 2i+1) or in halves (i, i + rot_dims / 2);
//   q and k divided by their root mean square (eps inside the root) and multiplied by a gain of d values shared by all
//   heads (null: no gain), after the rotation or, with `norm_first`, before it;
//   q multiplied by the query temperature 1 + coef * ln(floor((pos + 1) / every) + 1);
//   v = (1 - lambda) * v + lambda * v_first for a layer that mixes in an earlier layer's values of the same token;
//   score = scale * q.k, then cap * tanh(score / cap) if cap > 0, then minus slope[head] * (i - j) (a distance bias);
//   query at position i sees key j when j <= i and (window == 0 or i - j < window or j < keep_first); with `chunked`
//   the window is a chunk instead: j >= floor(i / window) * window;
//   softmax over the visible keys, whose denominator also holds exp(sink[head]) when sinks are given (a sink has no key
//   and no value and is neither scaled nor biased); weighted sum of the values.
// Everything after the loads is 32-bit; exponentials, tangents, sines, logarithms are the exact ones.
//
// Cache layout of one layer run: [page][kv head][slot in page][d + dv] — a token's key and value side by side.
#include "common.cuh"

namespace cib {

constexpr int kPrepWarps = 8;
constexpr int kPrepMaxPairsPerLane = 8;      // d and dv up to 512

// What the step before the attention does beside rotation and cache write; every pointer may be null.
struct PrepOptions {
    const float* bias;        // [H*d + G*d + G*dv] added to the packed rows
    const float* q_gain;      // [d] gain of the query heads' norm
    const float* k_gain;      // [d] gain of the key heads' norm
    int norm;                 // 0: no norm of q and k; 1: divided by their root mean square (times the gain, if any)
    int norm_first;           // the norm comes before the rotation
    int rot_half;             // rotation pairs are (i, i + rot_dims / 2) instead of (2i, 2i + 1)
    int has_temp;             // queries are multiplied by 1 + temp_coef * ln(floor((pos + 1) / temp_every) + 1)
    float temp_coef;
    int temp_every;
    int value_from_key;       // the packed rows are [q | k]: a token's value is its key as it stands before norm and rotation
    float rot_gain;           // cosine and sine are both multiplied by this (1: a pure rotation)
};

// One warp per (token, vector): H query heads, G key heads, G value heads of the packed rows [q | k | v] (with
// `value_from_key` there are no value vectors: the key's warp stores the value too).  C: pairs of values a lane holds
// (d <= 64 C).
template <typename T, int C>
__global__ void __launch_bounds__(kPrepWarps * 32)
window_attention_prep_kernel(T* __restrict__ qkv, int stride, const int* __restrict__ positions,
                             const int* __restrict__ slot_mapping, const float* __restrict__ freq, int rot_dims, float eps,
                             int H, int G, int d, int dv, const T* __restrict__ v_first, int v_first_stride,
                             AnyVec lambda, int has_lambda, T* __restrict__ cache, long long num_slots, int page_size,
                             int num_tokens, PrepOptions opt) {
    const int lane = threadIdx.x & 31;
    const int vectors = opt.value_from_key ? H + G : H + 2 * G;
    const long long w = (long long)blockIdx.x * kPrepWarps + (threadIdx.x >> 5);
    if (w >= (long long)num_tokens * vectors) return;
    const int t = (int)(w / vectors), vec = (int)(w % vectors);
    T* row = qkv + (size_t)t * stride;
    const int slot = slot_mapping ? slot_mapping[t] : -1;
    const bool store = cache && slot >= 0 && slot < num_slots;
    const int width = d + dv;
    if (vec >= H + G) {                                   // a value head: bias, mix and store
        const int g = vec - H - G;
        if (!store) return;
        const size_t off = (size_t)H * d + (size_t)G * d + (size_t)g * dv;
        const T* v = row + off;
        const float lam = has_lambda ? lambda[0] : 0.f;
        T* dst = cache + (((size_t)(slot / page_size) * G + g) * page_size + slot % page_size) * width + d;
        for (int i = lane; i < dv; i += 32) {
            float x = to_f32(v[i]);
            if (opt.bias) x += opt.bias[off + i];
            if (has_lambda) x = (1.f - lam) * x + lam * to_f32(v_first[(size_t)t * v_first_stride + (size_t)g * dv + i]);
            dst[i] = from_f32<T>(x);
        }
        return;
    }
    const bool is_key = vec >= H;
    const size_t off = is_key ? (size_t)H * d + (size_t)(vec - H) * d : (size_t)vec * d;
    T* x = row + off;
    const float* bias = opt.bias ? opt.bias + off : nullptr;
    const float* gain = is_key ? opt.k_gain : opt.q_gain;
    const int ipos = positions[t];
    const float pos = (float)ipos;
    const int half = rot_dims / 2;
    float a[C], b[C];
    // pair p of the lane's pairs: the rotation partners, or two neighbours of the part that is not rotated
    auto first_of = [&](int p) { return opt.rot_half && p < half ? p : 2 * p; };
    auto second_of = [&](int p) { return opt.rot_half && p < half ? p + half : 2 * p + 1; };
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int p = c * 32 + lane, e0 = first_of(p), e1 = second_of(p);
        a[c] = e0 < d ? to_f32(x[e0]) + (bias ? bias[e0] : 0.f) : 0.f;
        b[c] = e1 < d ? to_f32(x[e1]) + (bias ? bias[e1] : 0.f) : 0.f;
    }
    if (opt.value_from_key && is_key && store) {          // dv == d: the value is the key as projected
        T* vdst = cache + (((size_t)(slot / page_size) * G + (vec - H)) * page_size + slot % page_size) * width + d;
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const int p = c * 32 + lane, e0 = first_of(p), e1 = second_of(p);
            if (e0 < d) vdst[e0] = from_f32<T>(a[c]);
            if (e1 < d) vdst[e1] = from_f32<T>(b[c]);
        }
    }
    auto normalise = [&]() {
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < C; ++c) ss += a[c] * a[c] + b[c] * b[c];
        ss = warp_sum(ss);
        const float factor = 1.f / sqrtf(ss / (float)d + eps);
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const int p = c * 32 + lane, e0 = first_of(p), e1 = second_of(p);
            a[c] *= factor * (gain && e0 < d ? gain[e0] : 1.f);
            b[c] *= factor * (gain && e1 < d ? gain[e1] : 1.f);
        }
    };
    if (opt.norm && opt.norm_first) normalise();
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int p = c * 32 + lane;
        if (p < half && second_of(p) < d) {
            float sn, cs;
            sincosf(pos * freq[p], &sn, &cs);
            sn *= opt.rot_gain;
            cs *= opt.rot_gain;
            const float u = a[c], v = b[c];
            a[c] = u * cs - v * sn;
            b[c] = v * cs + u * sn;
        }
    }
    if (opt.norm && !opt.norm_first) normalise();
    if (opt.has_temp && !is_key) {
        const float temp = 1.f + opt.temp_coef * logf((float)((ipos + 1) / opt.temp_every + 1));
#pragma unroll
        for (int c = 0; c < C; ++c) { a[c] *= temp; b[c] *= temp; }
    }
    T* dst = x;
    if (is_key) {
        if (!store) return;
        dst = cache + (((size_t)(slot / page_size) * G + (vec - H)) * page_size + slot % page_size) * width;
    }
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int p = c * 32 + lane, e0 = first_of(p), e1 = second_of(p);
        if (e0 < d) dst[e0] = from_f32<T>(a[c]);
        if (e1 < d) dst[e1] = from_f32<T>(b[c]);
    }
}

constexpr int kWinWarps = 4;
constexpr int kWinMaxAcc = 16;               // dv up to 512

template <typename T>
__global__ void __launch_bounds__(kWinWarps * 32)
window_attention_generic_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                                const T* __restrict__ cache, int num_pages, int page_size,
                                const int* __restrict__ block_table, int table_stride, const int* __restrict__ positions,
                                const int* __restrict__ token_request, int H, int G, int d, int dv, float scale, float cap,
                                int window, int keep_first, int chunked, const float* __restrict__ slopes,
                                const float* __restrict__ sinks) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int head = blockIdx.y * kWinWarps + warp;
    if (head >= H) return;
    const int g = head / (H / G);
    float* qs = smem + warp * d;
    const int r = token_request[t];
    const int pos = positions[t];
    const int lo = window > 0 ? (chunked ? pos / window * window : max(0, pos - window + 1)) : 0;
    const float slope = slopes ? slopes[head] : 0.f;
    const int kept = window > 0 ? min(keep_first, lo) : 0;        // keys 0..kept-1 lie before the window and stay visible
    const int* table = block_table + (size_t)r * table_stride;
    const T* qp = q + (size_t)t * q_stride + (size_t)head * d;
    for (int i = lane; i < d; i += 32) qs[i] = to_f32(qp[i]);
    __syncwarp();

    float acc[kWinMaxAcc];
#pragma unroll
    for (int k = 0; k < kWinMaxAcc; ++k) acc[k] = 0.f;
    float m = -INFINITY, l = 0.f;
    const int width = d + dv;
    const float inv_cap = cap > 0.f ? 1.f / cap : 0.f;

    for (int seg = 0; seg < 2; ++seg) {
        const int begin = seg == 0 ? 0 : lo, end = seg == 0 ? kept : pos + 1;
        for (int c = begin; c < end; c += 32) {
            const int j = c + lane;
            float s = -INFINITY;
            const T* row = nullptr;
            if (j < end) {
                const int page = table[j / page_size];
                if (page >= 0 && page < num_pages) {
                    row = cache + (((size_t)page * G + g) * page_size + j % page_size) * width;
                    float dot = 0.f;
                    for (int i = 0; i < d; ++i) dot = fmaf(qs[i], to_f32(row[i]), dot);
                    s = dot * scale;
                    if (cap > 0.f) s = cap * tanhf(s * inv_cap);
                    s -= slope * (float)(pos - j);
                }
            }
            const float m_new = fmaxf(m, warp_max(s));
            if (m_new == -INFINITY) continue;                     // nothing visible in this chunk
            const float p = s == -INFINITY ? 0.f : expf(s - m_new);
            const float corr = m == -INFINITY ? 0.f : expf(m - m_new);
            l = l * corr + warp_sum(p);
            m = m_new;
#pragma unroll
            for (int k = 0; k < kWinMaxAcc; ++k) acc[k] *= corr;
            const int count = min(32, end - c);
            for (int jj = 0; jj < count; ++jj) {
                const float pj = __shfl_sync(0xffffffffu, p, jj);
                const T* vj = reinterpret_cast<const T*>(__shfl_sync(0xffffffffu, reinterpret_cast<uintptr_t>(row), jj));
                if (pj == 0.f || vj == nullptr) continue;
#pragma unroll
                for (int k = 0; k < kWinMaxAcc; ++k) {
                    const int i = k * 32 + lane;
                    if (i < dv) acc[k] = fmaf(pj, to_f32(vj[d + i]), acc[k]);
                }
            }
        }
    }
    if (sinks) {                                                  // the sink joins the denominator and nothing else
        const float sink = sinks[head];
        const float m_new = fmaxf(m, sink);
        const float corr = m == -INFINITY ? 0.f : expf(m - m_new);
        l = l * corr + expf(sink - m_new);
#pragma unroll
        for (int k = 0; k < kWinMaxAcc; ++k) acc[k] *= corr;
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    T* op = out + (size_t)t * out_stride + (size_t)head * dv;
#pragma unroll
    for (int k = 0; k < kWinMaxAcc; ++k) {
        const int i = k * 32 + lane;
        if (i < dv) op[i] = from_f32<T>(acc[k] * inv);
    }
}

}  // namespace cib

using namespace cib;

// bias (float32 [H*d + G*d + G*dv]), q_gain / k_gain (float32 [d]) may be null.  norm: 0 none, 1 root mean square (with
// the gains, if given); norm_first: before the rotation; rot_half: pairs (i, i + rot_dims / 2); has_temp: the query
// temperature with temp_coef and temp_every; value_from_key: rows are [q | k] and a token's cached value is its key before
// norm and rotation (dv == d); rot_gain: a factor on both cosine and sine.
extern "C" int cib_window_attention_prep(void* qkv, int dtype, int stride, const int* positions, const int* slot_mapping,
                                         const float* freq, int rot_dims, float eps, int H, int G, int d, int dv,
                                         const void* v_first, int v_first_stride, const void* lambda, int lambda_dtype,
                                         void* cache, long long num_slots, int page_size, int num_tokens,
                                         const float* bias, const float* q_gain, const float* k_gain, int norm, int norm_first,
                                         int rot_half, int has_temp, float temp_coef, int temp_every, int value_from_key,
                                         float rot_gain, cudaStream_t stream) {
    CIB_REQUIRE(H > 0 && G > 0 && H % G == 0 && d > 0 && dv > 0, "window_attention_prep: bad head counts or sizes");
    CIB_REQUIRE(d <= 64 * kPrepMaxPairsPerLane, "window_attention_prep: head size %d is beyond %d", d, 64 * kPrepMaxPairsPerLane);
    CIB_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= d && (rot_dims == 0 || freq), "window_attention_prep: bad rotation");
    CIB_REQUIRE((v_first == nullptr) == (lambda == nullptr), "window_attention_prep: mixing needs both the values and the factor");
    CIB_REQUIRE(!has_temp || temp_every > 0, "window_attention_prep: the query temperature needs a positive period");
    CIB_REQUIRE(!value_from_key || (d == dv && v_first == nullptr), "window_attention_prep: values taken from the keys have the keys' size and are not mixed");
    if (num_tokens == 0) return 0;
    const long long warps = (long long)num_tokens * (value_from_key ? H + G : H + 2 * G);
    const int blocks = (int)((warps + kPrepWarps - 1) / kPrepWarps);
    AnyVec lam{lambda, lambda_dtype == kBF16};
    PrepOptions opt{bias, q_gain, k_gain, norm, norm_first, rot_half, has_temp, temp_coef, temp_every, value_from_key, rot_gain};
#define CIB_PREP(T, C)                                                                                                        \
    window_attention_prep_kernel<T, C><<<blocks, kPrepWarps * 32, 0, stream>>>(                                               \
        (T*)qkv, stride, positions, slot_mapping, freq, rot_dims, eps, H, G, d, dv, (const T*)v_first, v_first_stride, lam,    \
        lambda != nullptr, (T*)cache, num_slots, page_size, num_tokens, opt)
#define CIB_PREP_BY_SIZE(T)                                                                                                   \
    {                                                                                                                         \
        if (d <= 64) CIB_PREP(T, 1);                                                                                          \
        else if (d <= 128) CIB_PREP(T, 2);                                                                                    \
        else if (d <= 256) CIB_PREP(T, 4);                                                                                    \
        else CIB_PREP(T, 8);                                                                                                  \
    }
    if (dtype == kF32) CIB_PREP_BY_SIZE(float)
    else if (dtype == kBF16) CIB_PREP_BY_SIZE(__nv_bfloat16)
    else CIB_REQUIRE(false, "window_attention_prep: bad dtype %d", dtype);
#undef CIB_PREP_BY_SIZE
#undef CIB_PREP
    CIB_LAUNCH_CHECK("window_attention_prep");
    return 0;
}

extern "C" int cib_window_attention_generic(const void* q, int dtype, int q_stride, void* out, int out_stride, const void* cache,
                                            int num_pages, int page_size, const int* block_table, int table_stride,
                                            const int* positions, const int* token_request, int num_tokens, int H, int G,
                                            int d, int dv, float scale, float cap, int window, int keep_first, int chunked,
                                            const float* slopes, const float* sinks, cudaStream_t stream) {
    CIB_REQUIRE(H > 0 && G > 0 && H % G == 0 && d > 0 && dv > 0, "window_attention: bad head counts or sizes");
    CIB_REQUIRE(dv <= 32 * kWinMaxAcc, "window_attention: value size %d is beyond %d", dv, 32 * kWinMaxAcc);
    CIB_REQUIRE(d <= 2048, "window_attention: head size %d is beyond 2048", d);
    CIB_REQUIRE(window >= 0 && keep_first >= 0, "window_attention: bad window");
    if (num_tokens == 0) return 0;
    dim3 grid(num_tokens, (H + kWinWarps - 1) / kWinWarps);
    const size_t smem = (size_t)kWinWarps * d * sizeof(float);
    if (dtype == kF32)
        window_attention_generic_kernel<float><<<grid, kWinWarps * 32, smem, stream>>>((const float*)q, q_stride, (float*)out, out_stride, (const float*)cache, num_pages, page_size, block_table, table_stride, positions, token_request, H, G, d, dv, scale, cap, window, keep_first, chunked, slopes, sinks);
    else if (dtype == kBF16)
        window_attention_generic_kernel<__nv_bfloat16><<<grid, kWinWarps * 32, smem, stream>>>((const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)cache, num_pages, page_size, block_table, table_stride, positions, token_request, H, G, d, dv, scale, cap, window, keep_first, chunked, slopes, sinks);
    else
        CIB_REQUIRE(false, "window_attention: bad dtype %d", dtype);
    CIB_LAUNCH_CHECK("window_attention_generic");
    return 0;
}

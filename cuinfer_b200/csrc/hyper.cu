// A residual of several streams (hyper-connections): every token keeps S rows x_0 .. x_{S-1} of W values in 32 bits.
// A sub-layer reads one row, u = sum_s in[s] x_s, and its output y is written back to all streams at once from the old
// ones, x_t <- sum_s mix[s][t] x_s + out[t] y.  One pass over a token's rows does, each part optional:
//   (1) the write of the sub-layer before (y, mix, out), in place;
//   (2) the read of the next sub-layer (in) and its RMS norm, u * rsqrt(mean(u^2) + eps) * gain, rounded once;
//   (3) u itself as a 32-bit row.
// Everything is 32-bit: coefficients, sums, the norm.  A block per token; a thread takes four, two or one neighbouring columns at a
// time (as W and the number of streams allow), whose S values live in registers; the
// row u waits in shared memory between the two passes of the norm.
//
// hyper_gather: for a few wanted tokens only, the sum of the streams after an outstanding write,
//   sum_t x_t' = sum_s (sum_t mix[s][t]) x_s + (sum_t out[t]) y, without touching the other tokens' rows.
#include "common.cuh"

namespace cib {

constexpr int kHyperMaxStreams = 16;

// V consecutive columns of a row as one access (V = 1, 2 or 4; the row starts on 4 V bytes and W is a multiple of V).
template <int V>
__device__ __forceinline__ void load_f32(const float* p, float (&v)[V]) {
    if constexpr (V == 4) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    } else if constexpr (V == 2) {
        const float2 t = *reinterpret_cast<const float2*>(p);
        v[0] = t.x; v[1] = t.y;
    } else {
        v[0] = *p;
    }
}
template <int V>
__device__ __forceinline__ void store_f32(float* p, const float (&v)[V]) {
    if constexpr (V == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    else if constexpr (V == 2) *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]);
    else *p = v[0];
}
template <int V>
__device__ __forceinline__ void load_any(const float* p, float (&v)[V]) { load_f32<V>(p, v); }
template <int V>
__device__ __forceinline__ void load_any(const __nv_bfloat16* p, float (&v)[V]) {
    if constexpr (V == 4) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    } else if constexpr (V == 2) {
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
        v[0] = a.x; v[1] = a.y;
    } else {
        v[0] = __bfloat162float(*p);
    }
}
template <int V>
__device__ __forceinline__ void store_any(float* p, const float (&v)[V]) { store_f32<V>(p, v); }
template <int V>
__device__ __forceinline__ void store_any(__nv_bfloat16* p, const float (&v)[V]) {
    if constexpr (V == 4) {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 raw;
        raw.x = *reinterpret_cast<const unsigned*>(&a);
        raw.y = *reinterpret_cast<const unsigned*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    } else if constexpr (V == 2) {
        *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v[0], v[1]);
    } else {
        *p = __float2bfloat16_rn(v[0]);
    }
}

// The largest block of hyper_stream_kernel<.., SM, V>: 2 * SM * V values of a thread's columns live in registers.
constexpr int hyper_block_cap(int SM, int V) { return SM * V > 16 || SM > 8 ? 256 : 512; }

template <typename TY, typename TO, int SM, int V>
__global__ void __launch_bounds__(hyper_block_cap(SM, V), hyper_block_cap(SM, V) == 512 ? 2 : 1)
hyper_stream_kernel(float* __restrict__ x, const TY* __restrict__ y, const float* __restrict__ mix,
                    const float* __restrict__ out_w, const float* __restrict__ in_w, AnyVec gain, int has_gain, float eps,
                    TO* __restrict__ normed, float* __restrict__ read_out, int S, int W) {
    extern __shared__ __align__(16) float u_row[];
    __shared__ float scratch[33];
    __shared__ float s_mix[kHyperMaxStreams * kHyperMaxStreams], s_out[kHyperMaxStreams], s_in[kHyperMaxStreams];
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < S * S; i += blockDim.x) s_mix[i] = y ? mix[i] : 0.f;
    for (int i = threadIdx.x; i < S; i += blockDim.x) {
        s_out[i] = y ? out_w[i] : 0.f;
        s_in[i] = in_w ? in_w[i] : 0.f;
    }
    __syncthreads();
    float* rows = x + (size_t)t * S * W;
    const bool reads = in_w != nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x * V; i < W; i += blockDim.x * V) {
        float old[SM][V], cur[SM][V];
#pragma unroll
        for (int s = 0; s < SM; ++s) {
            if (s < S) {
                load_f32<V>(rows + (size_t)s * W + i, old[s]);
            } else {
#pragma unroll
                for (int c = 0; c < V; ++c) old[s][c] = 0.f;
            }
        }
        if (y) {
            float yv[V];
            load_any<V>(y + (size_t)t * W + i, yv);
#pragma unroll
            for (int d = 0; d < SM; ++d) {
                if (d < S) {
#pragma unroll
                    for (int c = 0; c < V; ++c) {
                        float acc = 0.f;
#pragma unroll
                        for (int s = 0; s < SM; ++s)
                            if (s < S) acc = fmaf(s_mix[s * S + d], old[s][c], acc);
                        cur[d][c] = fmaf(s_out[d], yv[c], acc);
                    }
                    store_f32<V>(rows + (size_t)d * W + i, cur[d]);
                }
            }
        } else {
#pragma unroll
            for (int s = 0; s < SM; ++s)
#pragma unroll
                for (int c = 0; c < V; ++c) cur[s][c] = old[s][c];
        }
        if (reads) {
            float u[V];
#pragma unroll
            for (int c = 0; c < V; ++c) {
                u[c] = 0.f;
#pragma unroll
                for (int s = 0; s < SM; ++s)
                    if (s < S) u[c] = fmaf(s_in[s], cur[s][c], u[c]);
            }
            if (read_out) store_f32<V>(read_out + (size_t)t * W + i, u);
            if (normed) {
                store_f32<V>(u_row + i, u);
#pragma unroll
                for (int c = 0; c < V; ++c) ss = fmaf(u[c], u[c], ss);
            }
        }
    }
    if (!reads || !normed) return;
    ss = block_sum(ss, scratch);
    const float factor = 1.f / sqrtf(ss / (float)W + eps);
    for (int i = threadIdx.x * V; i < W; i += blockDim.x * V) {
        float u[V];
        load_f32<V>(u_row + i, u);
#pragma unroll
        for (int c = 0; c < V; ++c) u[c] = u[c] * factor * (has_gain ? gain[i + c] : 1.f);
        store_any<V>(normed + (size_t)t * W + i, u);
    }
}

template <typename TY, int V>
__global__ void __launch_bounds__(512)
hyper_gather_kernel(const float* __restrict__ x, const TY* __restrict__ y, const float* __restrict__ mix,
                    const float* __restrict__ out_w, const int* __restrict__ indices, float* __restrict__ out,
                    int S, int W, int num_tokens) {
    __shared__ float c[kHyperMaxStreams + 1];
    for (int j = threadIdx.x; j <= S; j += blockDim.x) {
        float v = 1.f;
        if (y) {
            v = 0.f;
            for (int d = 0; d < S; ++d) v += j < S ? mix[j * S + d] : out_w[d];
        } else if (j == S) {
            v = 0.f;
        }
        c[j] = v;
    }
    __syncthreads();
    const int t = indices[blockIdx.x];
    const bool outside = t < 0 || t >= num_tokens;
    const float* rows = x + (size_t)(outside ? 0 : t) * S * W;
    for (int i = threadIdx.x * V; i < W; i += blockDim.x * V) {
        float acc[V];
#pragma unroll
        for (int k = 0; k < V; ++k) acc[k] = 0.f;
        if (!outside) {
            if (y) {
                float yv[V];
                load_any<V>(y + (size_t)t * W + i, yv);
#pragma unroll
                for (int k = 0; k < V; ++k) acc[k] = c[S] * yv[k];
            }
            for (int s = 0; s < S; ++s) {
                float v[V];
                load_f32<V>(rows + (size_t)s * W + i, v);
#pragma unroll
                for (int k = 0; k < V; ++k) acc[k] = fmaf(c[s], v[k], acc[k]);
            }
        }
        store_f32<V>(out + (size_t)blockIdx.x * W + i, acc);
    }
}

// Threads for rows of W values taken V at a time: a multiple of 32 between 64 and `cap`.
static int hyper_threads(int W, int V, int cap = 512) {
    const int n = ((W + V - 1) / V + 31) / 32 * 32;
    return n < 64 ? 64 : n > cap ? cap : n;
}

template <typename TY, typename TO>
static int launch_hyper_stream(float* x, const void* y, const float* mix, const float* out_w, const float* in_w, AnyVec gain,
                               int has_gain, float eps, void* normed, float* read_out, int S, int W, int T, cudaStream_t stream) {
    // sixteen values of a thread's columns at most (four streams of four columns, eight of two), so that two blocks of 512
    // threads share an SM; the widest access that W allows
    const int V = S <= 4 && W % 4 == 0 ? 4 : S <= 8 && W % 2 == 0 ? 2 : 1;
    const size_t smem = normed ? (size_t)W * sizeof(float) : 0;
    // Few tokens (decode steps): the largest block, so that a row is done in the fewest dependent rounds of loads.  Many:
    // blocks of 256, of which the registers let three or more share an SM (measured at 8 192 tokens of 4 x 4 096:
    // one block of 512 threads per SM, 25 % of the warp slots, 3.7 TB/s).
    const bool many = T >= 2 * 148;
#define CIB_HS(SMv, Vv)                                                                                                          \
    {                                                                                                                            \
        static SmemLimit limit;                                                                                                  \
        if (smem > 48 * 1024)                                                                                                    \
            if (int rc = raise_smem_limit(limit, hyper_stream_kernel<TY, TO, SMv, Vv>, 200 * 1024, "hyper_stream")) return rc;   \
        hyper_stream_kernel<TY, TO, SMv, Vv><<<T, hyper_threads(W, Vv, many ? 256 : hyper_block_cap(SMv, Vv)), smem, stream>>>(x, (const TY*)y, mix, out_w, in_w, gain, has_gain,   \
                                                                           eps, (TO*)normed, read_out, S, W);                    \
    }
    if (V == 4) {
        if (S == 1) CIB_HS(1, 4)
        else if (S == 2) CIB_HS(2, 4)
        else CIB_HS(4, 4)
    } else if (V == 2) {
        if (S == 1) CIB_HS(1, 2)
        else if (S == 2) CIB_HS(2, 2)
        else if (S <= 4) CIB_HS(4, 2)
        else CIB_HS(8, 2)
    } else {
        if (S == 1) CIB_HS(1, 1)
        else if (S == 2) CIB_HS(2, 1)
        else if (S <= 4) CIB_HS(4, 1)
        else if (S <= 8) CIB_HS(8, 1)
        else CIB_HS(16, 1)
    }
#undef CIB_HS
    return 0;
}

}  // namespace cib

using namespace cib;

// x [T, S, W] float32, updated in place when y is given (then mix [S, S] (from, to) and out_w [S] are needed).  in_w [S]
// selects the read; with it, `normed` (out_dtype) gets the RMS norm of the read row times `gain` (a null gain is one) and
// `read_out` (float32) the read row itself.  y has dtype y_dtype.
extern "C" int cib_hyper_stream(float* x, const void* y, int y_dtype, const float* mix, const float* out_w, const float* in_w,
                                const void* gain, int gain_dtype, float eps, void* normed, int out_dtype, float* read_out,
                                int S, int W, int T, cudaStream_t stream) {
    CIB_REQUIRE(S >= 1 && S <= kHyperMaxStreams, "hyper_stream: %d streams are beyond %d", S, kHyperMaxStreams);
    CIB_REQUIRE(W > 0 && T >= 0 && (size_t)W * 4 <= 200 * 1024, "hyper_stream: bad sizes T=%d W=%d", T, W);
    CIB_REQUIRE(y == nullptr || (mix && out_w), "hyper_stream: a write needs its coefficients");
    CIB_REQUIRE((normed == nullptr && read_out == nullptr) || in_w, "hyper_stream: a read needs its coefficients");
    if (T == 0 || (y == nullptr && in_w == nullptr)) return 0;
    AnyVec g{gain, gain_dtype == kBF16};
    const int has_gain = gain != nullptr;
    const int yd = y ? y_dtype : kF32, od = normed ? out_dtype : kF32;
    int rc = -1;
    if (yd == kF32 && od == kF32) rc = launch_hyper_stream<float, float>(x, y, mix, out_w, in_w, g, has_gain, eps, normed, read_out, S, W, T, stream);
    else if (yd == kBF16 && od == kBF16) rc = launch_hyper_stream<__nv_bfloat16, __nv_bfloat16>(x, y, mix, out_w, in_w, g, has_gain, eps, normed, read_out, S, W, T, stream);
    else if (yd == kBF16 && od == kF32) rc = launch_hyper_stream<__nv_bfloat16, float>(x, y, mix, out_w, in_w, g, has_gain, eps, normed, read_out, S, W, T, stream);
    else if (yd == kF32 && od == kBF16) rc = launch_hyper_stream<float, __nv_bfloat16>(x, y, mix, out_w, in_w, g, has_gain, eps, normed, read_out, S, W, T, stream);
    else CIB_REQUIRE(false, "hyper_stream: bad dtypes %d / %d", y_dtype, out_dtype);
    if (rc) return rc;
    CIB_LAUNCH_CHECK("hyper_stream");
    return 0;
}

// out[r] = the sum of the streams of token indices[r] after the outstanding write (y, mix, out_w), or of the streams as
// they are when y is null.  An index outside 0..T-1 gives a zero row.
extern "C" int cib_hyper_gather(const float* x, const void* y, int y_dtype, const float* mix, const float* out_w,
                                const int* indices, float* out, int S, int W, int T, int rows, cudaStream_t stream) {
    CIB_REQUIRE(S >= 1 && S <= kHyperMaxStreams && W > 0 && T >= 0 && rows >= 0, "hyper_gather: bad sizes");
    CIB_REQUIRE(y == nullptr || (mix && out_w), "hyper_gather: a write needs its coefficients");
    if (rows == 0) return 0;
    const bool wide = W % 4 == 0;
    const int threads = hyper_threads(W, wide ? 4 : 1);
    if (y == nullptr || y_dtype == kF32) {
        if (wide) hyper_gather_kernel<float, 4><<<rows, threads, 0, stream>>>(x, (const float*)y, mix, out_w, indices, out, S, W, T);
        else hyper_gather_kernel<float, 1><<<rows, threads, 0, stream>>>(x, (const float*)y, mix, out_w, indices, out, S, W, T);
    } else if (y_dtype == kBF16) {
        if (wide) hyper_gather_kernel<__nv_bfloat16, 4><<<rows, threads, 0, stream>>>(x, (const __nv_bfloat16*)y, mix, out_w, indices, out, S, W, T);
        else hyper_gather_kernel<__nv_bfloat16, 1><<<rows, threads, 0, stream>>>(x, (const __nv_bfloat16*)y, mix, out_w, indices, out, S, W, T);
    } else {
        CIB_REQUIRE(false, "hyper_gather: bad dtype %d", y_dtype);
    }
    CIB_LAUNCH_CHECK("hyper_gather");
    return 0;
}

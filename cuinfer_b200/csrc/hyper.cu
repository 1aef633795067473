// A residual of several streams (hyper-connections): every token keeps S rows x_0 .. x_{S-1} of W values in 32 bits.
// A sub-layer reads one row, u = sum_s in[s] x_s, and its output y is written back to all streams at once from the old
// ones, x_t <- sum_s mix[s][t] x_s + out[t] y.  One pass over a token's rows does, each part optional:
//   (1) the write of the sub-layer before (y, mix, out), in place;
//   (2) the read of the next sub-layer (in) and its RMS norm, u * rsqrt(mean(u^2) + eps) * gain, rounded once;
//   (3) u itself as a 32-bit row.
// Everything is 32-bit: coefficients, sums, the norm.  A block per token; a column's S values live in registers, the
// row u in shared memory between the two passes of the norm.
//
// hyper_gather: for a few wanted tokens only, the sum of the streams after an outstanding write,
//   sum_t x_t' = sum_s (sum_t mix[s][t]) x_s + (sum_t out[t]) y, without touching the other tokens' rows.
#include "common.cuh"

namespace cib {

constexpr int kHyperMaxStreams = 8;

template <typename TY, typename TO, int SM>
__global__ void __launch_bounds__(256)
hyper_stream_kernel(float* __restrict__ x, const TY* __restrict__ y, const float* __restrict__ mix,
                    const float* __restrict__ out_w, const float* __restrict__ in_w, AnyVec gain, int has_gain, float eps,
                    TO* __restrict__ normed, float* __restrict__ read_out, int S, int W) {
    extern __shared__ float u_row[];
    __shared__ float scratch[33];
    __shared__ float s_mix[kHyperMaxStreams * kHyperMaxStreams], s_out[kHyperMaxStreams], s_in[kHyperMaxStreams];
    const int t = blockIdx.x;
    if (threadIdx.x < S * S) s_mix[threadIdx.x] = y ? mix[threadIdx.x] : 0.f;
    if (threadIdx.x < S) {
        s_out[threadIdx.x] = y ? out_w[threadIdx.x] : 0.f;
        s_in[threadIdx.x] = in_w ? in_w[threadIdx.x] : 0.f;
    }
    __syncthreads();
    float* rows = x + (size_t)t * S * W;
    const bool reads = in_w != nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        float old[SM], cur[SM];
#pragma unroll
        for (int s = 0; s < SM; ++s) old[s] = s < S ? rows[(size_t)s * W + i] : 0.f;
        if (y) {
            const float yv = to_f32(y[(size_t)t * W + i]);
#pragma unroll
            for (int d = 0; d < SM; ++d) {
                if (d < S) {
                    float acc = 0.f;
#pragma unroll
                    for (int s = 0; s < SM; ++s)
                        if (s < S) acc = fmaf(s_mix[s * S + d], old[s], acc);
                    cur[d] = fmaf(s_out[d], yv, acc);
                    rows[(size_t)d * W + i] = cur[d];
                }
            }
        } else {
#pragma unroll
            for (int s = 0; s < SM; ++s) cur[s] = old[s];
        }
        if (reads) {
            float u = 0.f;
#pragma unroll
            for (int s = 0; s < SM; ++s)
                if (s < S) u = fmaf(s_in[s], cur[s], u);
            if (read_out) read_out[(size_t)t * W + i] = u;
            if (normed) {
                u_row[i] = u;
                ss += u * u;
            }
        }
    }
    if (!reads || !normed) return;
    ss = block_sum(ss, scratch);
    const float factor = 1.f / sqrtf(ss / (float)W + eps);
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float g = has_gain ? gain[i] : 1.f;
        normed[(size_t)t * W + i] = from_f32<TO>(u_row[i] * factor * g);
    }
}

template <typename TY>
__global__ void hyper_gather_kernel(const float* __restrict__ x, const TY* __restrict__ y, const float* __restrict__ mix,
                                    const float* __restrict__ out_w, const int* __restrict__ indices, float* __restrict__ out,
                                    int S, int W, int num_tokens) {
    __shared__ float c[kHyperMaxStreams + 1];
    if (threadIdx.x <= S) {
        float v = 1.f;
        if (y) {
            v = 0.f;
            for (int d = 0; d < S; ++d) v += threadIdx.x < S ? mix[threadIdx.x * S + d] : out_w[d];
        } else if (threadIdx.x == S) {
            v = 0.f;
        }
        c[threadIdx.x] = v;
    }
    __syncthreads();
    const int t = indices[blockIdx.x];
    if (t < 0 || t >= num_tokens) {
        for (int i = threadIdx.x; i < W; i += blockDim.x) out[(size_t)blockIdx.x * W + i] = 0.f;
        return;
    }
    const float* rows = x + (size_t)t * S * W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        float acc = y ? c[S] * to_f32(y[(size_t)t * W + i]) : 0.f;
        for (int s = 0; s < S; ++s) acc = fmaf(c[s], rows[(size_t)s * W + i], acc);
        out[(size_t)blockIdx.x * W + i] = acc;
    }
}

template <typename TY, typename TO>
static int launch_hyper_stream(float* x, const void* y, const float* mix, const float* out_w, const float* in_w, AnyVec gain,
                               int has_gain, float eps, void* normed, float* read_out, int S, int W, int T, cudaStream_t stream) {
    const int threads = W >= 256 ? 256 : ((W + 31) / 32 * 32 < 64 ? 64 : (W + 31) / 32 * 32);
    const size_t smem = normed ? (size_t)W * sizeof(float) : 0;
#define CIB_HS(SMv)                                                                                                             \
    {                                                                                                                           \
        static SmemLimit limit;                                                                                                 \
        if (smem > 48 * 1024)                                                                                                   \
            if (int rc = raise_smem_limit(limit, hyper_stream_kernel<TY, TO, SMv>, 200 * 1024, "hyper_stream")) return rc;      \
        hyper_stream_kernel<TY, TO, SMv><<<T, threads, smem, stream>>>(x, (const TY*)y, mix, out_w, in_w, gain, has_gain, eps, \
                                                                       (TO*)normed, read_out, S, W);                            \
    }
    if (S == 1) CIB_HS(1)
    else if (S == 2) CIB_HS(2)
    else if (S <= 4) CIB_HS(4)
    else CIB_HS(8)
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
    const int threads = W >= 256 ? 256 : 64;
    if (y == nullptr || y_dtype == kF32)
        hyper_gather_kernel<float><<<rows, threads, 0, stream>>>(x, (const float*)y, mix, out_w, indices, out, S, W, T);
    else if (y_dtype == kBF16)
        hyper_gather_kernel<__nv_bfloat16><<<rows, threads, 0, stream>>>(x, (const __nv_bfloat16*)y, mix, out_w, indices, out, S, W, T);
    else
        CIB_REQUIRE(false, "hyper_gather: bad dtype %d", y_dtype);
    CIB_LAUNCH_CHECK("hyper_gather");
    return 0;
}

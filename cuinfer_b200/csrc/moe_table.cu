// Mixture of gated experts whose choice is a table lookup: expert_table[token id][0..top-1] names the experts of a
// token, each with the same weight.  An expert is down_e( silu(gate_e h) * (up_e h) ), no biases.
//
// The simple kernels: every (token, choice) streams its expert's rows — a matrix-vector product per token, which is
// what a decode step needs (a token's experts are read once) and the 32-bit path.  Two launches:
//   gate_up : act[t, k, j] = silu(Wg[e][j, :] . h_t) * (Wu[e][j, :] . h_t),  e = table[ids[t], k]
//   down    : out[t, i]    = base[t, i] + weight * sum_k Wd[e_k][i, :] . act[t, k, :]
// Dots and the gate are 32-bit with the exact exponential; act and out are rounded once to the rows' type.
// Weights: gate_up [E][2 ff][W] (gate rows, then up rows), down [E][W][ff].  A table entry outside 0..E-1 contributes
// nothing.  `base` (another feed-forward's output, a shared expert's say) may be null.
//
// The same kernels serve experts chosen by a router: `ids` null means that the table is indexed by the row itself
// (table[t][k] = the k-th expert chosen for row t), `weights[t][k]` (32-bit, may be null) replaces the uniform weight,
// and `act_kind` 1 selects the clamped gate  g = min(gate, limit), u = clamp(up, -limit, limit),
// act = g * sigmoid(1.702 g) * (u + 1)  instead of silu(gate) * up.  `act_kind` 2 is an expert WITHOUT a gate,
// down_e( relu(up_e h)^2 ): its first matrix is [E][ff][W] (up rows only).  `base_gate` (32-bit, one number per row, `base_gate_stride` apart; may
// be null): base is multiplied by sigmoid(base_gate[t]) as it is added (a shared expert with a gate of its own).
#include "common.cuh"

namespace cib {

constexpr int kMoeWarps = 8;
// outputs a block computes: 32 for rows of up to 2 048 values (more blocks: a decode step of eight tokens is 80 / 150 us a
// call instead of 94 / 170 at widths of 1 024 / 2 048), 64 for longer ones (a block's copy of its input row is shared by more)
static inline int moe_outs_per_block(int width) { return width > 2048 ? 64 : 32; }

struct ExpertAct {
    int kind;        // 0: silu(gate) * up;  1: the clamped gate described above;  2: no gate, relu(up)^2;  -1: nothing
    float limit;
    __host__ __device__ __forceinline__ bool gated() const { return kind == 0 || kind == 1; }
    // an expert without a gate: what becomes of its one product
    __device__ __forceinline__ float single(float u) const {
        if (kind == 2) {
            u = fmaxf(u, 0.f);
            return u * u;
        }
        return u;
    }
    __device__ __forceinline__ float operator()(float g, float u) const {
        if (kind == 1) {
            g = fminf(g, limit);
            u = fminf(fmaxf(u, -limit), limit);
            return g / (1.f + expf(-1.702f * g)) * (u + 1.f);
        }
        return g / (1.f + expf(-g)) * u;
    }
};

template <typename T>
__device__ __forceinline__ float dot_row(const T* __restrict__ w, const float* __restrict__ x, int n, int lane) {
    float s = 0.f;
    for (int i = lane; i < n; i += 32) s = fmaf(to_f32(w[i]), x[i], s);
    return warp_sum(s);
}
// bfloat16 rows of a multiple of 8 values that start on a 16-byte boundary: a lane reads 16 bytes at a time (a warp
// 512 bytes per load instead of 64), four loads issued before the first is used.
template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const __nv_bfloat16* __restrict__ w, const float* __restrict__ x, int n,
                                                        int lane) {
    float s = 0.f;
    if ((n & 7) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0) {
        const uint4* w8 = reinterpret_cast<const uint4*>(w);
        const int chunks = n >> 3;
        int c = lane;
        for (; c + 96 < chunks; c += 128) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = __ldg(w8 + c + 32 * u);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[u]);
                const float* xs = x + (c + 32 * u) * 8;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    s = fmaf(__low2float(h[k]), xs[2 * k], s);
                    s = fmaf(__high2float(h[k]), xs[2 * k + 1], s);
                }
            }
        }
        for (; c < chunks; c += 32) {
            const uint4 v = __ldg(w8 + c);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
            const float* xs = x + c * 8;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                s = fmaf(__low2float(h[k]), xs[2 * k], s);
                s = fmaf(__high2float(h[k]), xs[2 * k + 1], s);
            }
        }
    } else {
        for (int i = lane; i < n; i += 32) s = fmaf(__bfloat162float(w[i]), x[i], s);
    }
    return warp_sum(s);
}

// Two rows at once, each against its own vector: the loads of both rows are issued before either is used, so a lane
// keeps eight 16-byte loads in flight instead of four (a decode step has too few warps an SM for four to fill the
// memory pipe: two rows at a time took a call of the large experts from 180 to 107 us).  Every row is summed in the
// order `dot_row` sums it, so the results are the same to the last bit.
template <typename T>
__device__ __forceinline__ void dot_rows2(const T* __restrict__ w0, const float* __restrict__ x0, const T* __restrict__ w1,
                                          const float* __restrict__ x1, int n, int lane, float& r0, float& r1) {
    r0 = dot_row(w0, x0, n, lane);
    r1 = dot_row(w1, x1, n, lane);
}
__device__ __forceinline__ float dot_chunk(const uint4& v, const float* __restrict__ xs, float s) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        s = fmaf(__low2float(h[k]), xs[2 * k], s);
        s = fmaf(__high2float(h[k]), xs[2 * k + 1], s);
    }
    return s;
}
template <>
__device__ __forceinline__ void dot_rows2<__nv_bfloat16>(const __nv_bfloat16* __restrict__ w0, const float* __restrict__ x0,
                                                         const __nv_bfloat16* __restrict__ w1, const float* __restrict__ x1, int n,
                                                         int lane, float& r0, float& r1) {
    if ((n & 7) != 0 || ((reinterpret_cast<uintptr_t>(w0) | reinterpret_cast<uintptr_t>(w1)) & 15) != 0) {
        r0 = dot_row(w0, x0, n, lane);
        r1 = dot_row(w1, x1, n, lane);
        return;
    }
    const uint4* a8 = reinterpret_cast<const uint4*>(w0);
    const uint4* b8 = reinterpret_cast<const uint4*>(w1);
    const int chunks = n >> 3;
    float s0 = 0.f, s1 = 0.f;
    int c = lane;
    for (; c + 96 < chunks; c += 128) {
        uint4 a[4], b[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) a[u] = __ldg(a8 + c + 32 * u);
#pragma unroll
        for (int u = 0; u < 4; ++u) b[u] = __ldg(b8 + c + 32 * u);
#pragma unroll
        for (int u = 0; u < 4; ++u) s0 = dot_chunk(a[u], x0 + (c + 32 * u) * 8, s0);
#pragma unroll
        for (int u = 0; u < 4; ++u) s1 = dot_chunk(b[u], x1 + (c + 32 * u) * 8, s1);
    }
    for (; c < chunks; c += 32) {
        const uint4 a = __ldg(a8 + c), b = __ldg(b8 + c);
        s0 = dot_chunk(a, x0 + c * 8, s0);
        s1 = dot_chunk(b, x1 + c * 8, s1);
    }
    r0 = warp_sum(s0);
    r1 = warp_sum(s1);
}

template <typename T>
__global__ void __launch_bounds__(kMoeWarps * 32)
moe_table_gate_up_kernel(const T* __restrict__ h, int h_stride, const int* __restrict__ ids,
                         const int* __restrict__ table, int vocab, int top, int experts,
                         const T* __restrict__ gate_up, T* __restrict__ act, int width, int ff, ExpertAct fn, int outs) {
    extern __shared__ float hs[];
    const int t = blockIdx.x / top, k = blockIdx.x % top;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < width; i += blockDim.x) hs[i] = to_f32(h[(size_t)t * h_stride + i]);
    __syncthreads();
    const int id = ids ? ids[t] : t;
    const int e = (id >= 0 && id < vocab) ? table[(size_t)id * top + k] : -1;
    const bool ok = e >= 0 && e < experts;
    const bool gated = fn.gated();
    const T* wg = gate_up + (size_t)(ok ? e : 0) * (gated ? 2 : 1) * ff * width;
    const T* wu = wg + (size_t)ff * width;
    const int j0 = blockIdx.y * outs, j_end = min(ff, j0 + outs);
    T* dst = act + ((size_t)t * top + k) * ff;
    if (gated) {                                      // a gate row and its up row together
        for (int j = j0 + warp; j < j_end; j += kMoeWarps) {
            float g = 0.f, u = 0.f;
            if (ok) dot_rows2(wg + (size_t)j * width, hs, wu + (size_t)j * width, hs, width, lane, g, u);
            if (lane == 0) dst[j] = from_f32<T>(ok ? fn(g, u) : 0.f);
        }
        return;
    }
    for (int j = j0 + warp; j < j_end; j += 2 * kMoeWarps) {          // two rows of the one matrix together
        const int j2 = j + kMoeWarps;
        float a = 0.f, b = 0.f;
        if (ok) {
            if (j2 < j_end) dot_rows2(wg + (size_t)j * width, hs, wg + (size_t)j2 * width, hs, width, lane, a, b);
            else a = dot_row(wg + (size_t)j * width, hs, width, lane);
        }
        if (lane == 0) {
            dst[j] = from_f32<T>(ok ? fn.single(a) : 0.f);
            if (j2 < j_end) dst[j2] = from_f32<T>(ok ? fn.single(b) : 0.f);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kMoeWarps * 32)
moe_table_down_kernel(const T* __restrict__ act, const int* __restrict__ ids, const int* __restrict__ table, int vocab,
                      int top, int experts, const T* __restrict__ down, const T* __restrict__ base, int base_stride,
                      float weight, const float* __restrict__ weights, const float* __restrict__ base_gate, int base_gate_stride,
                      T* __restrict__ out, int width, int ff, int outs) {
    extern __shared__ float as[];                       // [top][ff]
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < top * ff; i += blockDim.x) as[i] = to_f32(act[(size_t)t * top * ff + i]);
    __syncthreads();
    const int id = ids ? ids[t] : t;
    const bool id_ok = id >= 0 && id < vocab;
    const int i0 = blockIdx.y * outs, i_end = min(width, i0 + outs);
    const float bg = base && base_gate ? 1.f / (1.f + expf(-base_gate[(size_t)t * base_gate_stride])) : 1.f;
    for (int i = i0 + warp; i < i_end; i += 2 * kMoeWarps) {           // two outputs together
        const int i2 = i + kMoeWarps;
        float sum[2] = {0.f, 0.f};
        for (int k = 0; k < top; ++k) {
            const int e = id_ok ? table[(size_t)id * top + k] : -1;
            if (e < 0 || e >= experts) continue;
            float d0, d1 = 0.f;
            if (i2 < i_end) dot_rows2(down + ((size_t)e * width + i) * ff, as + k * ff, down + ((size_t)e * width + i2) * ff, as + k * ff, ff, lane, d0, d1);
            else d0 = dot_row(down + ((size_t)e * width + i) * ff, as + k * ff, ff, lane);
            const float wk = weights ? weights[(size_t)t * top + k] : 1.f;
            sum[0] += wk * d0;
            sum[1] += wk * d1;
        }
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int o = r == 0 ? i : i2;
                if (o >= i_end) continue;
                float v = weights ? sum[r] : sum[r] * weight;
                if (base) v += to_f32(base[(size_t)t * base_stride + o]) * bg;
                out[(size_t)t * width + o] = from_f32<T>(v);
            }
        }
    }
}

}  // namespace cib

using namespace cib;

extern "C" int cib_moe_table_gate_up(const void* h, int h_stride, int dtype, const int* ids, const int* table, int vocab,
                                     int top, int experts, const void* gate_up, void* act, int num_tokens, int width,
                                     int ff, int act_kind, float limit, cudaStream_t stream) {
    CIB_REQUIRE(num_tokens >= 0 && top > 0 && experts > 0 && width > 0 && ff > 0 && vocab > 0, "moe_table: bad sizes");
    CIB_REQUIRE(width <= 12 * 1024, "moe_table: width %d too large for this kernel", width);
    if (num_tokens == 0) return 0;
    const int outs = moe_outs_per_block(width);
    dim3 grid(num_tokens * top, (ff + outs - 1) / outs);
    const size_t smem = (size_t)width * sizeof(float);
    if (dtype == kF32)
        moe_table_gate_up_kernel<float><<<grid, kMoeWarps * 32, smem, stream>>>((const float*)h, h_stride, ids, table, vocab, top, experts, (const float*)gate_up, (float*)act, width, ff, ExpertAct{act_kind, limit}, outs);
    else if (dtype == kBF16)
        moe_table_gate_up_kernel<__nv_bfloat16><<<grid, kMoeWarps * 32, smem, stream>>>((const __nv_bfloat16*)h, h_stride, ids, table, vocab, top, experts, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)act, width, ff, ExpertAct{act_kind, limit}, outs);
    else
        CIB_REQUIRE(false, "moe_table: unsupported dtype %d", dtype);
    CIB_LAUNCH_CHECK("moe_table_gate_up");
    return 0;
}

extern "C" int cib_moe_table_down(const void* act, int dtype, const int* ids, const int* table, int vocab, int top,
                                  int experts, const void* down, const void* base, int base_stride, float weight,
                                  const float* weights, const float* base_gate, int base_gate_stride, void* out, int num_tokens,
                                  int width, int ff, cudaStream_t stream) {
    CIB_REQUIRE(num_tokens >= 0 && top > 0 && experts > 0 && width > 0 && ff > 0 && vocab > 0, "moe_table: bad sizes");
    CIB_REQUIRE((size_t)top * ff <= 50 * 1024, "moe_table: %d x %d activations too large for this kernel", top, ff);
    if (num_tokens == 0) return 0;
    const int outs = moe_outs_per_block(width);
    dim3 grid(num_tokens, (width + outs - 1) / outs);
    const size_t smem = (size_t)top * ff * sizeof(float);        // a token's activations of all its experts, 32-bit
    if (smem > 48 * 1024) {
        static SmemLimit limit_f32, limit_bf16;
        const int rc = dtype == kF32 ? raise_smem_limit(limit_f32, moe_table_down_kernel<float>, 200 * 1024, "moe_table_down")
                                     : raise_smem_limit(limit_bf16, moe_table_down_kernel<__nv_bfloat16>, 200 * 1024, "moe_table_down");
        if (rc != 0) return rc;
    }
    if (dtype == kF32)
        moe_table_down_kernel<float><<<grid, kMoeWarps * 32, smem, stream>>>((const float*)act, ids, table, vocab, top, experts, (const float*)down, (const float*)base, base_stride, weight, weights, base_gate, base_gate_stride, (float*)out, width, ff, outs);
    else if (dtype == kBF16)
        moe_table_down_kernel<__nv_bfloat16><<<grid, kMoeWarps * 32, smem, stream>>>((const __nv_bfloat16*)act, ids, table, vocab, top, experts, (const __nv_bfloat16*)down, (const __nv_bfloat16*)base, base_stride, weight, weights, base_gate, base_gate_stride, (__nv_bfloat16*)out, width, ff, outs);
    else
        CIB_REQUIRE(false, "moe_table: unsupported dtype %d", dtype);
    CIB_LAUNCH_CHECK("moe_table_down");
    return 0;
}

// ---- many tokens: rows sorted by expert, then one tensor-core product per expert group ---------------------------------
// A prompt portion gives every expert many rows, so the experts' matrices are worth reading once per 64-row tile
// instead of once per token.  Everything is decided on the device (the step may be replayed from a CUDA graph):
//   route   : count the (token, choice) slots of every expert, lay the slots out expert by expert, and list the
//             64-row tiles of every group (one block; the order of slots inside a group is whatever the atomics give,
//             which changes no result: every row is computed on its own)
//   grouped : out rows of a tile = A rows x W_e^T on mma.sync m16n8k16 — with A gathered through the slot list and
//             silu(gate) * up as the epilogue for the first product, plain for the second
//   combine : out[t] = base[t] + weight * sum over the token's slots of its down-projected rows
#include "mma_utils.cuh"

namespace cib {

constexpr int kGM = 64, kGN = 64, kGK = 32, kGStages = 3, kGLd = kGK + 8;

__global__ void __launch_bounds__(1024)
moe_route_kernel(const int* __restrict__ ids, const int* __restrict__ table, int vocab, int top, int experts, int slots,
                 int* __restrict__ sorted_slot, int* __restrict__ slot_pos, int* __restrict__ offsets,
                 int* __restrict__ tile_expert, int* __restrict__ tile_row0, int* __restrict__ num_tiles, int max_tiles) {
    extern __shared__ int route_s[];                    // counts[E], cursor[E], start[E + 1]
    int* counts = route_s;
    int* cursor = route_s + experts;
    int* start = route_s + 2 * experts;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) { counts[e] = 0; cursor[e] = 0; }
    __syncthreads();
    auto expert_of = [&](int slot) {
        const int id = ids ? ids[slot / top] : slot / top;
        const int e = (id >= 0 && id < vocab) ? table[(size_t)id * top + slot % top] : -1;
        return (e >= 0 && e < experts) ? e : -1;
    };
    for (int s = threadIdx.x; s < slots; s += blockDim.x) {
        const int e = expert_of(s);
        if (e >= 0) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tiles = 0;
        for (int e = 0; e < experts; ++e) {
            start[e] = at;
            for (int r = 0; r < counts[e] && tiles < max_tiles; r += kGM) {
                tile_expert[tiles] = e;
                tile_row0[tiles] = at + r;
                ++tiles;
            }
            at += counts[e];
        }
        start[experts] = at;
        *num_tiles = tiles;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= experts; e += blockDim.x) offsets[e] = start[e];
    for (int s = threadIdx.x; s < slots; s += blockDim.x) {
        const int e = expert_of(s);
        int at = -1;
        if (e >= 0) {
            at = start[e] + atomicAdd(&cursor[e], 1);
            sorted_slot[at] = s;
        }
        slot_pos[s] = at;
    }
}

// out[r, n] for the rows r of one tile of one expert's group; w: [E][N_total][K] with the expert's rows `w_expert`
// elements apart.  GATED: columns j and N + j of the expert are gate and up, out[r, j] = silu(gate) * up, out has N
// columns.  Otherwise out[r, j] for 128 columns a CTA, through `fn.single` (an expert without a gate squares its ReLU
// there; the second product passes kind -1).  `gather`: row r of A is a[(gather[r] / top)]; else a[r].
template <bool GATED>
__global__ void __launch_bounds__(128)
moe_grouped_gemm_kernel(const __nv_bfloat16* __restrict__ a, int lda, const int* __restrict__ gather, int top,
                        const __nv_bfloat16* __restrict__ w, long long w_expert, __nv_bfloat16* __restrict__ out, int ldo,
                        const int* __restrict__ offsets, const int* __restrict__ tile_expert,
                        const int* __restrict__ tile_row0, const int* __restrict__ num_tiles, int N, int K, ExpertAct fn) {
    __shared__ __align__(16) __nv_bfloat16 sA[kGStages][kGM][kGLd];
    __shared__ __align__(16) __nv_bfloat16 sB[kGStages][2][kGN][kGLd];
    if ((int)blockIdx.x >= *num_tiles) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int e = tile_expert[blockIdx.x];
    const int r0 = tile_row0[blockIdx.x];
    const int rows = min(kGM, offsets[e + 1] - r0);
    const int n0 = blockIdx.y * (GATED ? kGN : 2 * kGN);
    const int second = GATED ? N : kGN;                       // where the second 64-column tile's weight rows start
    const __nv_bfloat16* we = w + (size_t)e * w_expert;

    // what this thread copies per stage: two 16-byte chunks of A, four of B
    const __nv_bfloat16* a_src[2];
    bool a_ok[2];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const int idx = tid + c * 128, row = idx >> 2;
        a_ok[c] = row < rows;
        const int src_row = a_ok[c] ? (gather ? gather[r0 + row] / top : r0 + row) : 0;
        a_src[c] = a + (size_t)src_row * lda + (idx & 3) * 8;
    }
    const __nv_bfloat16* b_src[4];
    bool b_ok[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const int idx = tid + c * 128, half = idx >> 8, row = (idx >> 2) & 63;
        const int col = n0 + row;                              // output column of this weight row within its half
        b_ok[c] = GATED ? col < N : col + half * kGN < N;
        b_src[c] = we + (size_t)(b_ok[c] ? half * second + col : 0) * K + (idx & 3) * 8;
    }
    auto load = [&](int stage, int k0) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int idx = tid + c * 128;
            cp_async16(&sA[stage][idx >> 2][(idx & 3) * 8], a_src[c] + k0, a_ok[c]);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int idx = tid + c * 128;
            cp_async16(&sB[stage][idx >> 8][(idx >> 2) & 63][(idx & 3) * 8], b_src[c] + k0, b_ok[c]);
        }
    };

    float acc[2][kGN / 8][4];
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int i = 0; i < kGN / 8; ++i) { acc[h][i][0] = acc[h][i][1] = acc[h][i][2] = acc[h][i][3] = 0.f; }

    const int steps = K / kGK;
#pragma unroll
    for (int s = 0; s < kGStages - 1; ++s) {
        if (s < steps) load(s, s * kGK);
        cp_async_commit();
    }
    const int mat = lane >> 3, rr = lane & 7;
    for (int ks = 0; ks < steps; ++ks) {
        cp_async_wait<kGStages - 2>();
        __syncthreads();
        if (ks + kGStages - 1 < steps) load((ks + kGStages - 1) % kGStages, (ks + kGStages - 1) * kGK);
        cp_async_commit();
        const int st = ks % kGStages;
#pragma unroll
        for (int kk = 0; kk < kGK / 16; ++kk) {
            uint32_t af[4];
            ldmatrix_x4(af, smem_u32(&sA[st][warp * 16 + (mat & 1) * 8 + rr][kk * 16 + (mat >> 1) * 8]));
#pragma unroll
            for (int h = 0; h < 2; ++h) {
#pragma unroll
                for (int np = 0; np < kGN / 16; ++np) {
                    uint32_t b[4];
                    ldmatrix_x4(b, smem_u32(&sB[st][h][np * 16 + (mat >> 1) * 8 + rr][kk * 16 + (mat & 1) * 8]));
                    mma_bf16_16816(acc[h][2 * np], af, b[0], b[1]);
                    mma_bf16_16816(acc[h][2 * np + 1], af, b[2], b[3]);
                }
            }
        }
    }
    cp_async_wait<0>();

    const int qrow = lane >> 2, quad = lane & 3;
#pragma unroll
    for (int hrow = 0; hrow < 2; ++hrow) {
        const int row = warp * 16 + qrow + 8 * hrow;
        if (row >= rows) continue;
        __nv_bfloat16* dst = out + (size_t)(r0 + row) * ldo;
        if (GATED) {
#pragma unroll
            for (int nt = 0; nt < kGN / 8; ++nt) {
                const int col = n0 + nt * 8 + quad * 2;
                const float g0 = acc[0][nt][2 * hrow], g1 = acc[0][nt][2 * hrow + 1];
                const float v0 = fn(g0, acc[1][nt][2 * hrow]);
                const float v1 = fn(g1, acc[1][nt][2 * hrow + 1]);
                if (col + 1 < N) *reinterpret_cast<uint32_t*>(dst + col) = pack_bf16(v0, v1);
                else if (col < N) dst[col] = __float2bfloat16_rn(v0);
            }
        } else {
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int nt = 0; nt < kGN / 8; ++nt) {
                    const int col = n0 + h * kGN + nt * 8 + quad * 2;
                    const float v0 = fn.single(acc[h][nt][2 * hrow]), v1 = fn.single(acc[h][nt][2 * hrow + 1]);
                    if (col + 1 < N) *reinterpret_cast<uint32_t*>(dst + col) = pack_bf16(v0, v1);
                    else if (col < N) dst[col] = __float2bfloat16_rn(v0);
                }
        }
    }
}

__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ slot_pos, int top,
                                   const __nv_bfloat16* __restrict__ base, int base_stride, float weight,
                                   const float* __restrict__ weights, const float* __restrict__ base_gate, int base_gate_stride,
                                   __nv_bfloat16* __restrict__ out, int width) {
    const int t = blockIdx.x;
    const float bg = base && base_gate ? 1.f / (1.f + expf(-base_gate[(size_t)t * base_gate_stride])) : 1.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float sum = 0.f;
        for (int k = 0; k < top; ++k) {
            const int at = slot_pos[t * top + k];
            if (at >= 0) sum += (weights ? weights[t * top + k] : 1.f) * __bfloat162float(y[(size_t)at * width + i]);
        }
        float v = weights ? sum : sum * weight;
        if (base) v += __bfloat162float(base[(size_t)t * base_stride + i]) * bg;
        out[(size_t)t * width + i] = __float2bfloat16_rn(v);
    }
}

}  // namespace cib

extern "C" int cib_moe_table_grouped_supports(int width, int ff, int experts) {
    return width % cib::kGK == 0 && ff % cib::kGK == 0 && experts > 0 && experts <= 4096;
}

// Integers of workspace the grouped path needs: sorted slots, their inverse, group offsets, the tile list, the tile count.
extern "C" long long cib_moe_table_grouped_workspace_ints(int num_tokens, int top, int experts) {
    const long long slots = (long long)num_tokens * top;
    const long long max_tiles = (slots + cib::kGM - 1) / cib::kGM + experts;
    return 2 * slots + (experts + 1) + 2 * max_tiles + 1;
}

// bfloat16 only.  act: [T * top, ff] and y: [T * top, width] scratch rows; ints: see above.
extern "C" int cib_moe_table_grouped(const void* h, int h_stride, const int* ids, const int* table, int vocab, int top,
                                     int experts, const void* gate_up, const void* down, const void* base, int base_stride,
                                     float weight, const float* weights, const float* base_gate, int base_gate_stride, void* out,
                                     void* act, void* y, int* ints, int num_tokens, int width, int ff, int act_kind, float limit,
                                     cudaStream_t stream) {
    using namespace cib;
    CIB_REQUIRE(num_tokens >= 0 && top > 0 && vocab > 0, "moe_table_grouped: bad sizes");
    CIB_REQUIRE(cib_moe_table_grouped_supports(width, ff, experts), "moe_table_grouped: width %d / ff %d / %d experts are not taken", width, ff, experts);
    CIB_REQUIRE(h_stride % 8 == 0, "moe_table_grouped: rows must start on 16-byte boundaries");
    if (num_tokens == 0) return 0;
    const long long slots64 = (long long)num_tokens * top;
    CIB_REQUIRE(slots64 < (1ll << 30), "moe_table_grouped: too many rows");
    const int slots = (int)slots64;
    const int max_tiles = (slots + kGM - 1) / kGM + experts;
    int* sorted_slot = ints;
    int* slot_pos = sorted_slot + slots;
    int* offsets = slot_pos + slots;
    int* tile_expert = offsets + experts + 1;
    int* tile_row0 = tile_expert + max_tiles;
    int* num_tiles = tile_row0 + max_tiles;
    moe_route_kernel<<<1, 1024, (size_t)(3 * experts + 1) * sizeof(int), stream>>>(ids, table, vocab, top, experts, slots, sorted_slot,
                                                                                   slot_pos, offsets, tile_expert, tile_row0,
                                                                                   num_tiles, max_tiles);
    CIB_LAUNCH_CHECK("moe_route");
    const ExpertAct fn{act_kind, limit};
    if (fn.gated()) {
        dim3 g1(max_tiles, (ff + kGN - 1) / kGN);
        moe_grouped_gemm_kernel<true><<<g1, 128, 0, stream>>>((const __nv_bfloat16*)h, h_stride, sorted_slot, top,
                                                              (const __nv_bfloat16*)gate_up, (long long)2 * ff * width,
                                                              (__nv_bfloat16*)act, ff, offsets, tile_expert, tile_row0, num_tiles, ff, width, fn);
    } else {
        dim3 g1(max_tiles, (ff + 2 * kGN - 1) / (2 * kGN));
        moe_grouped_gemm_kernel<false><<<g1, 128, 0, stream>>>((const __nv_bfloat16*)h, h_stride, sorted_slot, top,
                                                               (const __nv_bfloat16*)gate_up, (long long)ff * width,
                                                               (__nv_bfloat16*)act, ff, offsets, tile_expert, tile_row0, num_tiles, ff, width, fn);
    }
    CIB_LAUNCH_CHECK("moe_grouped_gate_up");
    dim3 g2(max_tiles, (width + 2 * kGN - 1) / (2 * kGN));
    moe_grouped_gemm_kernel<false><<<g2, 128, 0, stream>>>((const __nv_bfloat16*)act, ff, nullptr, top, (const __nv_bfloat16*)down,
                                                           (long long)width * ff, (__nv_bfloat16*)y, width, offsets, tile_expert,
                                                           tile_row0, num_tiles, width, ff, ExpertAct{-1, 0.f});
    CIB_LAUNCH_CHECK("moe_grouped_down");
    moe_combine_kernel<<<num_tokens, 256, 0, stream>>>((const __nv_bfloat16*)y, slot_pos, top, (const __nv_bfloat16*)base, base_stride,
                                                       weight, weights, base_gate, base_gate_stride, (__nv_bfloat16*)out, width);
    CIB_LAUNCH_CHECK("moe_combine");
    return 0;
}

// Attention with a capped score and a window that keeps the first tokens, on the tensor cores (bfloat16), for steps
// that bring prompt portions (alone or beside decoded tokens).  Same arithmetic as the all-sizes kernel in
// attention_window.cu; same tiling as this package's paged prefill kernel (attention_prefill.cu): the rows of a tile are
// (query token x query head of one kv head) folded together, 64 rows a CTA (16 a warp), 64-key tiles copied row by row
// with cp.async into two swizzled shared-memory stages, ldmatrix + mma.sync m16n8k16 with 32-bit accumulation, running
// softmax in base 2 with the scores in registers.  What differs:
//   * keys (DK values) and values (DV values) have sizes of their own and lie side by side in a cache row
//     [page][kv head][slot][DK + DV];
//   * score = scale * q.k, then cap * tanh(score / cap) when cap > 0 (32-bit; tanh through the exponential);
//   * a query at position i sees key j when j <= i and (window == 0 or i - j < window or j < keep_first): a tile walks
//     the key tiles of the kept tokens that lie before its window (keys 0 .. min(keep_first, window start) - 1) and then
//     those from its window's start to its last query;
//   * optional: a distance bias, score -= slope[head] * (i - j); a window that is a chunk (`chunked`: key j is seen
//     when floor(j / window) == floor(i / window)); sinks, one score per head that joins the softmax's denominator and
//     nothing else.
// The softmax weights are rounded to bfloat16 for the second product; everything before that is 32-bit.
#include "mma_utils.cuh"

namespace cib {

constexpr int kWmWarps = 4;
constexpr int kWmM = 64;     // rows per CTA
constexpr int kWmN = 64;     // keys per tile
constexpr int kWmStages = 2;

// where chunk `c` (8 values) of row `r` lies in a shared-memory row of CH chunks: conflict-free for ldmatrix
template <int CH>
__device__ __forceinline__ int wm_swz(int r, int c) {
    if (CH >= 8) return c ^ (r & 7);
    return c ^ ((r >> 1) & (CH - 1));
}

// Two threads copy one key/value row of a tile, half of its 16-byte chunks each, from the page whose number the caller
// has looked up a tile ahead (the table lookup, the row's address and the copy are three dependent trips otherwise).
template <int DK, int DV>
__device__ __forceinline__ void wm_load_kv_row(__nv_bfloat16* sK, __nv_bfloat16* sV, const __nv_bfloat16* cache, int page, int j,
                                               int page_size, int num_pages, int nkv, int kvh, int row, int half) {
    constexpr int kCK = DK / 8, kCV = DV / 8, kC = kCK + kCV, kHalf = kC / 2;
    const bool valid = page >= 0 && page < num_pages;
    const __nv_bfloat16* src = cache + (((size_t)(valid ? page : 0) * nkv + kvh) * page_size + (valid ? j % page_size : 0)) * (DK + DV);
#pragma unroll
    for (int c = 0; c < kHalf; ++c) {
        const int chunk = half * kHalf + c;
        __nv_bfloat16* dst = chunk < kCK ? sK + row * DK + wm_swz<kCK>(row, chunk) * 8
                                         : sV + row * DV + wm_swz<kCV>(row, chunk - kCK) * 8;
        cp_async16(dst, src + chunk * 8, valid);
    }
}

template <int DK, int DV, bool kFewRows>
__global__ void __launch_bounds__(kWmWarps * 32, 3)
window_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out,
                            int out_stride, const __nv_bfloat16* __restrict__ cache, int num_pages, int page_size,
                            const int* __restrict__ block_table, int table_stride,
                            const int* __restrict__ query_start_loc, const int* __restrict__ seq_lens,
                            int num_requests, int nq, int nkv, float scale, float cap, int window, int keep_first,
                            int num_splits, float* __restrict__ partial, int chunked, const float* __restrict__ slopes,
                            const float* __restrict__ sinks) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ int s_req, s_tile, s_q0, s_n, s_seq;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quad = lane & 3, qrow = lane >> 2;
    const int kvh = blockIdx.y;
    const int g = nq / nkv;
    constexpr int kCK = DK / 8, kCV = DV / 8;
    constexpr float kLog2e = 1.4426950408889634f;

    // Which request and which of its row tiles this CTA has: the first warp reads 32 requests' bounds at once and finds
    // the tile by a prefix sum over its lanes (one trip to memory instead of one per request before this one); the
    // request's start, token count and length come back from the same trip.
    if (warp == 0) {
        int t = blockIdx.x, found = num_requests, tile = 0, q0_f = 0, n_f = 0, seq_f = 0;
        for (int base = 0; base < num_requests; base += 32) {
            const int rr = base + lane;
            int q0_l = 0, n_l = 0, seq_l = 0;
            if (rr < num_requests) {
                q0_l = query_start_loc[rr];
                n_l = query_start_loc[rr + 1] - q0_l;
                seq_l = seq_lens[rr];
            }
            const int tiles = n_l > 0 ? (n_l * g + kWmM - 1) / kWmM : 0;
            int incl = tiles;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl += v;
            }
            const int excl = incl - tiles;
            const unsigned hit = __ballot_sync(0xffffffffu, t >= excl && t < incl);
            if (hit) {
                const int src = __ffs(hit) - 1;
                found = base + src;
                tile = t - __shfl_sync(0xffffffffu, excl, src);
                q0_f = __shfl_sync(0xffffffffu, q0_l, src);
                n_f = __shfl_sync(0xffffffffu, n_l, src);
                seq_f = __shfl_sync(0xffffffffu, seq_l, src);
                break;
            }
            t -= __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) {
            s_req = found;
            s_tile = tile;
            s_q0 = q0_f;
            s_n = n_f;
            s_seq = seq_f;
        }
    }
    __syncthreads();
    const int r = s_req;
    if (r >= num_requests) return;
    const int q0 = s_q0;
    const int n = s_n;
    const int seq_len = s_seq;
    const int rows_total = n * g;
    const int row0 = s_tile * kWmM;
    // A tile with rows in its first sixteen only (a decode step; a short portion; a request's last rows): the four warps
    // share out the KEYS of every key tile instead, sixteen each against the same rows, and merge at the end.
    // (Compiled in only for launches whose requests all have so few rows: the row-parallel form pays nothing for it.)
    const bool split_keys = kFewRows && rows_total - row0 <= 16;
    const int wrow = split_keys ? 0 : warp * 16;      // this warp's first row of the tile
    const int* table = block_table + (size_t)r * table_stride;

    constexpr int kStageElems = kWmN * (DK + DV);
    __nv_bfloat16* sKV = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* sQ = sKV + (size_t)kStageElems;            // the query tile borrows stage 1 (DK <= DK + DV)
    auto stage_k = [&](int s) { return sKV + (size_t)s * kStageElems; };
    auto stage_v = [&](int s) { return sKV + (size_t)s * kStageElems + kWmN * DK; };

    // ---- key tiles: the kept tokens before the window, then the window up to the last query ----
    const int last_row = min(row0 + kWmM, rows_total) - 1;
    const int pos_first = seq_len - n + row0 / g;
    const int pos_last = seq_len - n + last_row / g;
    auto window_start = [&](int pos) { return window > 0 ? (chunked ? pos / window * window : max(0, pos - window + 1)) : 0; };
    int k_lo = window_start(pos_first);
    k_lo = k_lo / kWmN * kWmN;
    const int k_hi = pos_last + 1;
    const int kept_end = window > 0 ? min(keep_first, k_lo) : 0;
    const int kept_tiles = (kept_end + kWmN - 1) / kWmN;
    const int num_tiles = kept_tiles + (k_hi - k_lo + kWmN - 1) / kWmN;
    auto tile_key0 = [&](int t) { return t < kept_tiles ? t * kWmN : k_lo + (t - kept_tiles) * kWmN; };
    auto tile_end = [&](int t) { return t < kept_tiles ? kept_end : k_hi; };
    // with several splits (decode steps over long windows) this CTA walks a share of the key tiles and leaves its
    // running maximum, sum and unnormalised output for the merge kernel
    const int t_begin = (int)((long long)num_tiles * blockIdx.z / num_splits);
    const int t_end = (int)((long long)num_tiles * (blockIdx.z + 1) / num_splits);
    // this thread's key row of every tile, and the page that holds it (-1: past the tile's end, or no such tile)
    const int my_row = tid >> 1, my_half = tid & 1;
    auto lookup = [&](int t) {
        if (t >= t_end) return -1;
        const int j = tile_key0(t) + my_row;
        return j < tile_end(t) ? table[j / page_size] : -1;
    };
    auto load_tile = [&](int t, int page) {
        wm_load_kv_row<DK, DV>(stage_k((t - t_begin) % kWmStages), stage_v((t - t_begin) % kWmStages), cache, page, tile_key0(t) + my_row, page_size,
                               num_pages, nkv, kvh, my_row, my_half);
    };
    const int page_first = lookup(t_begin);
    int page_next = lookup(t_begin + 1);

    {
        for (int idx = tid; idx < kWmM * kCK; idx += kWmWarps * 32) {
            const int row = idx / kCK, chunk = idx % kCK;
            const int grow = row0 + row;
            const bool valid = grow < rows_total;
            const int tl = valid ? grow / g : 0, hi = valid ? grow % g : 0;
            const __nv_bfloat16* src = q + (size_t)(q0 + tl) * q_stride + (size_t)(kvh * g + hi) * DK + chunk * 8;
            cp_async16(sQ + row * DK + wm_swz<kCK>(row, chunk) * 8, src, valid);
        }
        cp_async_commit();
    }
    if (t_begin < t_end) load_tile(t_begin, page_first);
    cp_async_commit();

    cp_async_wait<1>();
    __syncthreads();
    uint32_t qf[DK / 16][4];
    {
        const int mat = lane >> 3, rr = lane & 7;
        const int row = wrow + (mat & 1) * 8 + rr;
#pragma unroll
        for (int kt = 0; kt < DK / 16; ++kt) {
            const int chunk = 2 * kt + (mat >> 1);
            ldmatrix_x4(qf[kt], smem_u32(sQ + row * DK + wm_swz<kCK>(row, chunk) * 8));
        }
    }
    __syncthreads();          // every warp has its query fragments: stage 1 may now take keys and values
    int pos_row[2], lo_row[2];
    bool row_ok[2];
    float slope_row[2];          // the distance bias of the row's head, in base-2 units
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int grow = row0 + wrow + qrow + 8 * h;
        row_ok[h] = grow < rows_total;
        pos_row[h] = row_ok[h] ? seq_len - n + grow / g : -1;
        lo_row[h] = row_ok[h] ? window_start(pos_row[h]) : 0;
        slope_row[h] = slopes && row_ok[h] ? slopes[kvh * g + grow % g] * kLog2e : 0.f;
    }

    // first and last position among this warp's rows: a key tile that every one of them sees whole needs no mask
    const int warp_row_first = row0 + wrow, warp_row_last = min(row0 + wrow + 15, rows_total - 1);
    const bool warp_has_rows = warp_row_first < rows_total;
    const int warp_pos_min = seq_len - n + (warp_has_rows ? warp_row_first : 0) / g;
    const int warp_pos_max = seq_len - n + (warp_has_rows ? warp_row_last : 0) / g;
    const bool warp_full = warp_row_first + 15 < rows_total;      // no row of the warp is padding

    float o[DV / 8][4];
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY};
    float l_run[2] = {0.f, 0.f};
    const float inv_cap = cap > 0.f ? 1.f / cap : 0.f;

    for (int t = t_begin; t < t_end; ++t) {
        const int key0 = tile_key0(t);
        const bool kept_tile = t < kept_tiles;
        if (t + 1 < t_end) load_tile(t + 1, page_next);
        cp_async_commit();
        page_next = lookup(t + 2);
        cp_async_wait<1>();
        __syncthreads();
        const __nv_bfloat16* sK = stage_k((t - t_begin) % kWmStages);      // the first tile of a CTA goes to stage 0: the queries borrow stage 1
        const __nv_bfloat16* sV = stage_v((t - t_begin) % kWmStages);

        float s[kWmN / 8][4];
#pragma unroll
        for (int nt = 0; nt < kWmN / 8; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f; }
        {
            const int mat = lane >> 3, rr = lane & 7;
#pragma unroll
            for (int kt = 0; kt < DK / 16; ++kt) {
#pragma unroll
                for (int np = 0; np < kWmN / 16; ++np) {
                    if (split_keys && np != warp) continue;
                    const int krow = np * 16 + (mat >> 1) * 8 + rr;
                    const int chunk = 2 * kt + (mat & 1);
                    uint32_t b[4];
                    ldmatrix_x4(b, smem_u32(sK + krow * DK + wm_swz<kCK>(krow, chunk) * 8));
                    mma_bf16_16816(s[2 * np], qf[kt], b[0], b[1]);
                    mma_bf16_16816(s[2 * np + 1], qf[kt], b[2], b[3]);
                }
            }
        }
        const bool need_mask = !warp_full || (kept_tile ? key0 + kWmN > kept_end
                                                        : (key0 + kWmN - 1 > warp_pos_min || (window > 0 && key0 < window_start(warp_pos_max))));
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < kWmN / 8; ++nt) {
            if (split_keys && (nt >> 1) != warp) {
                s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = -INFINITY;
                continue;
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int h = e >> 1;
                float v = s[nt][e] * scale;
                if (cap > 0.f) {
                    // cap * tanh(v / cap) = cap * (1 - 2 / (exp(2 v / cap) + 1)); the exponent is bounded so that it stays finite
                    const float x = fminf(fmaxf(2.f * v * inv_cap, -60.f), 60.f);
                    v = cap * (1.f - __fdividef(2.f, __expf(x) + 1.f));
                }
                v *= kLog2e;
                const int key = key0 + nt * 8 + quad * 2 + (e & 1);
                if (slopes) v -= slope_row[h] * (float)(pos_row[h] - key);
                if (need_mask) {
                    const int pos = pos_row[h];
                    const bool vis = kept_tile ? (key < kept_end && pos >= 0)
                                               : (key <= pos && (window <= 0 || key >= lo_row[h] || key < keep_first));
                    v = vis ? v : -INFINITY;
                }
                s[nt][e] = v;
                mx[h] = fmaxf(mx[h], v);
            }
        }
        float corr[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float m_new = fmaxf(m_run[h], mx[h]);
            corr[h] = m_run[h] == -INFINITY ? 0.f : exp2f(m_run[h] - m_new);
            m_run[h] = m_new;
            l_run[h] *= corr[h];
        }
#pragma unroll
        for (int nt = 0; nt < kWmN / 8; ++nt) {
            if (split_keys && (nt >> 1) != warp) continue;      // their weights are not read: the second product skips them
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float mref = m_run[e >> 1];
                const float p = (s[nt][e] == -INFINITY || mref == -INFINITY) ? 0.f : exp2f(s[nt][e] - mref);
                s[nt][e] = p;
                l_run[e >> 1] += p;
            }
        }
#pragma unroll
        for (int i = 0; i < DV / 8; ++i) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
        {
            const int mat = lane >> 3, rr = lane & 7;
#pragma unroll
            for (int kp = 0; kp < kWmN / 16; ++kp) {
                if (split_keys && kp != warp) continue;
                uint32_t pf[4];
                pf[0] = pack_bf16(s[2 * kp][0], s[2 * kp][1]);
                pf[1] = pack_bf16(s[2 * kp][2], s[2 * kp][3]);
                pf[2] = pack_bf16(s[2 * kp + 1][0], s[2 * kp + 1][1]);
                pf[3] = pack_bf16(s[2 * kp + 1][2], s[2 * kp + 1][3]);
                const int vrow = kp * 16 + (mat & 1) * 8 + rr;
#pragma unroll
                for (int nt = 0; nt < DV / 16; ++nt) {
                    const int chunk = 2 * nt + (mat >> 1);
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, smem_u32(sV + vrow * DV + wm_swz<kCV>(vrow, chunk) * 8));
                    mma_bf16_16816(o[2 * nt], pf, b[0], b[1]);
                    mma_bf16_16816(o[2 * nt + 1], pf, b[2], b[3]);
                }
            }
        }
        __syncthreads();      // every warp is done with this stage before it is filled again
    }
    cp_async_wait<0>();

    if (split_keys) {
        // Warps 1 to 3 leave their running maxima, sums and outputs in shared memory, lane by lane (the fragments of all
        // four warps cover the same rows and columns); the first warp folds them into its own and goes on alone.
        constexpr int kVals = DV / 2 + 4;
        float* scratch = reinterpret_cast<float*>(smem_raw);      // 3 x kVals x 32 floats: the stages are free by now
        if (warp > 0) {
            float* mine = scratch + (size_t)(warp - 1) * kVals * 32 + lane;
#pragma unroll
            for (int i = 0; i < DV / 8; ++i) {
#pragma unroll
                for (int e = 0; e < 4; ++e) mine[(i * 4 + e) * 32] = o[i][e];
            }
            mine[(DV / 2) * 32] = m_run[0];
            mine[(DV / 2 + 1) * 32] = m_run[1];
            mine[(DV / 2 + 2) * 32] = l_run[0];
            mine[(DV / 2 + 3) * 32] = l_run[1];
        }
        __syncthreads();
        if (warp > 0) return;
#pragma unroll 1
        for (int w = 0; w < kWmWarps - 1; ++w) {
            const float* theirs = scratch + (size_t)w * kVals * 32 + lane;
            float mine_f[2], theirs_f[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float m_w = theirs[(DV / 2 + h) * 32];
                const float m_new = fmaxf(m_run[h], m_w);
                mine_f[h] = m_run[h] == -INFINITY ? 0.f : exp2f(m_run[h] - m_new);
                theirs_f[h] = m_w == -INFINITY ? 0.f : exp2f(m_w - m_new);
                m_run[h] = m_new;
                l_run[h] = l_run[h] * mine_f[h] + theirs[(DV / 2 + 2 + h) * 32] * theirs_f[h];
            }
#pragma unroll
            for (int i = 0; i < DV / 8; ++i) {
#pragma unroll
                for (int e = 0; e < 4; ++e) o[i][e] = o[i][e] * mine_f[e >> 1] + theirs[(i * 4 + e) * 32] * theirs_f[e >> 1];
            }
        }
    }

#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float l = l_run[h];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        if (!row_ok[h]) continue;
        const int grow = row0 + wrow + qrow + 8 * h;
        const int tl = grow / g, hi = grow % g;
        float rescale = 1.f;
        if (sinks && num_splits == 1) {                // the sink joins the denominator (the merge kernel adds it otherwise)
            const float sink = sinks[kvh * g + hi] * kLog2e;
            const float m_new = fmaxf(m_run[h], sink);
            rescale = m_run[h] == -INFINITY ? 0.f : exp2f(m_run[h] - m_new);
            l = l * rescale + exp2f(sink - m_new);
        }
        const float inv = (l > 0.f ? 1.f / l : 0.f) * rescale;
        if (num_splits > 1) {
            float* dst = partial + (((size_t)(q0 + tl) * nq + kvh * g + hi) * num_splits + blockIdx.z) * (DV + 2);
#pragma unroll
            for (int nt = 0; nt < DV / 8; ++nt) {
                dst[nt * 8 + quad * 2] = o[nt][2 * h];
                dst[nt * 8 + quad * 2 + 1] = o[nt][2 * h + 1];
            }
            if (quad == 0) {
                dst[DV] = m_run[h];
                dst[DV + 1] = l;
            }
            continue;
        }
        __nv_bfloat16* dst = out + (size_t)(q0 + tl) * out_stride + (size_t)(kvh * g + hi) * DV;
#pragma unroll
        for (int nt = 0; nt < DV / 8; ++nt) {
            *reinterpret_cast<uint32_t*>(dst + nt * 8 + quad * 2) = pack_bf16(o[nt][2 * h] * inv, o[nt][2 * h + 1] * inv);
        }
    }
}

// out[row] = sum_i o_i 2^(m_i - M) / sum_i l_i 2^(m_i - M) over the splits' partial results; a warp per (token, head).
// Lane i holds split i's (and split i + 32's) maximum and sum, so the weights come from one trip to memory and a
// reduction over the lanes; the columns then read all splits' outputs with the weights handed round by shuffles.
__global__ void window_attention_merge_kernel(const float* __restrict__ partial, int num_splits, int dv,
                                              __nv_bfloat16* __restrict__ out, int out_stride, int nq, int rows,
                                              const float* __restrict__ sinks) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float* base = partial + (size_t)row * num_splits * (dv + 2);
    float m_l[2], l_l[2], w_l[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int i = lane + 32 * k;
        m_l[k] = i < num_splits ? base[(size_t)i * (dv + 2) + dv] : -INFINITY;
        l_l[k] = i < num_splits ? base[(size_t)i * (dv + 2) + dv + 1] : 0.f;
    }
    const float sink = sinks ? sinks[row % nq] * 1.4426950408889634f : -INFINITY;     // maxima are in base-2 units
    float M = fmaxf(fmaxf(m_l[0], m_l[1]), sink);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, d));
    float L = 0.f;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        w_l[k] = m_l[k] == -INFINITY ? 0.f : exp2f(m_l[k] - M);
        L += l_l[k] * w_l[k];
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) L += __shfl_xor_sync(0xffffffffu, L, d);
    if (sinks) L += exp2f(sink - M);
    const float inv = L > 0.f ? 1.f / L : 0.f;
    __nv_bfloat16* dst = out + (size_t)(row / nq) * out_stride + (size_t)(row % nq) * dv;
    // every lane walks every split, so that the shuffles meet; a split's four loads of a lane are issued together
    // (value sizes up to 128, which is all the tensor-core kernel takes), whatever the weight, and count only if it is not zero
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 2
    for (int i = 0; i < num_splits; ++i) {
        const float w = __shfl_sync(0xffffffffu, i < 32 ? w_l[0] : w_l[1], i & 31);
        const float* src = base + (size_t)i * (dv + 2);
        float v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = lane + 32 * k < dv ? src[lane + 32 * k] : 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[k] = w != 0.f ? fmaf(v[k], w, acc[k]) : acc[k];
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        if (lane + 32 * k < dv) dst[lane + 32 * k] = __float2bfloat16_rn(acc[k] * inv);
    }
}

template <int DK, int DV>
static int launch_window_mma(const void* q, int q_stride, void* out, int out_stride, const void* cache, int num_pages,
                             int page_size, const int* block_table, int table_stride, const int* query_start_loc,
                             const int* seq_lens, int num_requests, int num_tiles, int nq, int nkv, float scale, float cap,
                             int window, int keep_first, int num_splits, float* partial, int num_tokens, int chunked,
                             bool few_rows, const float* slopes, const float* sinks, cudaStream_t stream) {
    const size_t smem = (size_t)(kWmStages * kWmN * (DK + DV)) * sizeof(__nv_bfloat16);
    static SmemLimit limit, limit_few;
    auto kernel = few_rows ? window_attention_mma_kernel<DK, DV, true> : window_attention_mma_kernel<DK, DV, false>;
    if (int rc = raise_smem_limit(few_rows ? limit_few : limit, kernel, smem, "window_attention_mma")) return rc;
    dim3 grid(num_tiles, nkv, num_splits);
    kernel<<<grid, kWmWarps * 32, smem, stream>>>(
        (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)cache, num_pages,
        page_size, block_table, table_stride, query_start_loc, seq_lens, num_requests, nq, nkv, scale, cap, window, keep_first,
        num_splits, partial, chunked, slopes, sinks);
    CIB_LAUNCH_CHECK("window_attention_mma");
    if (num_splits > 1) {
        const int rows = num_tokens * nq;
        window_attention_merge_kernel<<<(rows + 7) / 8, 256, 0, stream>>>(partial, num_splits, DV, (__nv_bfloat16*)out, out_stride, nq, rows, sinks);
        CIB_LAUNCH_CHECK("window_attention_merge");
    }
    return 0;
}

}  // namespace cib

using namespace cib;

extern "C" int cib_window_attention_mma_supports(int dim, int vdim, int nq, int nkv) {
    return (dim == 64 || dim == 128) && (vdim == 32 || vdim == 64 || vdim == 128) && nkv > 0 && nq % nkv == 0;
}

// num_tiles: the sum over requests of ceil(tokens_r * (nq / nkv) / 64), or any upper bound of it (CTAs that find no
// tile leave).  num_splits > 1: every row tile's key tiles are shared out to so many CTAs, which leave float32 partial
// results in `partial` ([tokens * nq][num_splits][vdim + 2]: output, running maximum, sum) for a second kernel to merge.
// chunked: the window is a chunk (keys from floor(i / window) * window on); slopes, sinks: float32 [nq] or null.
// few_rows: no request has more than 16 rows (tokens * nq / nkv) in this launch, e.g. a decode step: the form whose
// warps share out a tile's keys instead of its rows runs (any tile with more rows still takes the row-parallel path).
extern "C" int cib_window_attention_mma(const void* q, int q_stride, void* out, int out_stride, const void* cache,
                                        int num_pages, int page_size, const int* block_table, int table_stride,
                                        const int* query_start_loc, const int* seq_lens, int num_requests, int num_tiles,
                                        int nq, int nkv, int dim, int vdim, float scale, float cap, int window,
                                        int keep_first, int num_splits, float* partial, int num_tokens, int chunked,
                                        int few_rows, const float* slopes, const float* sinks, cudaStream_t stream) {
    CIB_REQUIRE(cib_window_attention_mma_supports(dim, vdim, nq, nkv), "window_attention_mma: sizes %d / %d are not taken by this kernel", dim, vdim);
    CIB_REQUIRE(num_requests >= 0 && num_tiles >= 0 && nkv <= 65535, "window_attention_mma: bad sizes");
    CIB_REQUIRE(num_splits >= 1 && num_splits <= 64 && (num_splits == 1 || partial), "window_attention_mma: %d splits need room for their partial results", num_splits);
    CIB_REQUIRE(page_size > 0 && num_pages > 0 && table_stride > 0 && window >= 0 && keep_first >= 0, "window_attention_mma: bad cache geometry");
    CIB_REQUIRE(q_stride % 8 == 0 && ((uintptr_t)q % 16) == 0 && out_stride % 2 == 0 && ((uintptr_t)out % 4) == 0 && ((uintptr_t)cache % 16) == 0,
                "window_attention_mma: q and cache rows must be 16-byte aligned and out rows 4-byte aligned");
    if (num_requests == 0 || num_tiles == 0) return 0;
#define CIB_WM(DKv, DVv)                                                                                                     \
    if (dim == DKv && vdim == DVv)                                                                                           \
        return launch_window_mma<DKv, DVv>(q, q_stride, out, out_stride, cache, num_pages, page_size, block_table, table_stride, \
                                           query_start_loc, seq_lens, num_requests, num_tiles, nq, nkv, scale, cap, window,     \
                                           keep_first, num_splits, partial, num_tokens, chunked, few_rows != 0, slopes, sinks, stream)
    CIB_WM(64, 32);
    CIB_WM(64, 64);
    CIB_WM(64, 128);
    CIB_WM(128, 32);
    CIB_WM(128, 64);
    CIB_WM(128, 128);
#undef CIB_WM
    CIB_REQUIRE(false, "window_attention_mma: no kernel for %d / %d", dim, vdim);
    return -1;
}

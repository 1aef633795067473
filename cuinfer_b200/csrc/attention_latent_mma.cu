// Attention over cached latent rows [c (rk) | k_rot (dr)] on the tensor cores (mma.sync m16n8k16, bfloat16 operands,
// 32-bit accumulation), for prompt portions, mixed batches and decode steps alike.  What it computes is stated at
// the head of attention_latent.cu; this file is the bfloat16 path for rk and dr that are multiples of 16, rk <= 512.
//
// All heads read the same rows, so a CTA's query tile of M = 64 rows is (tokens x heads) of ONE request: HB = 2^k heads
// side by side (k smallest with HB >= min(H, M)) times M / HB consecutive tokens; a decode step's single token fills the
// tile with its heads, and with 32 heads or fewer a decode step runs tiles of M = 32 rows (no idle rows, and two CTAs
// to an SM).  Keys come in tiles of 32 rows through two cp.async stages; S = Q K^T runs over all rk + dr
// columns, O += P V over the first rk columns of the same shared-memory tile (the values ARE the latents).  A warp owns
// 16 rows; for rk > 256 eight warps share them in pairs, each computing S again and keeping half of the value columns
// (128 accumulator registers a thread).  The query's rotary part is encoded as the tile is loaded; softmax statistics
// are 32-bit in the log2 domain; the sink starts a row's running maximum and counts once in its sum.  With a window
// (query i sees key j when 0 <= i - j < window) a tile starts at the first key tile its first token sees and masks both
// edges; cosine and sine of the rotation are multiplied by `rot_gain`.
//
// gridDim.z > 1 splits a tile's keys over CTAs (decode steps: few rows, long contexts).  Each split then writes its
// running maximum, its sum and its unnormalised rows to a scratch buffer and a second kernel merges them with the sink.
#include "common.cuh"
#include "mma_utils.cuh"

namespace cib {

constexpr int kLmN = 32;       // keys of a tile (a query tile has 16 * RG rows)
constexpr float kLog2e = 1.4426950408889634f;

template <int RKH, int CS, int RG>
__global__ void __launch_bounds__(32 * RG * CS)
latent_attention_mma_kernel(const __nv_bfloat16* __restrict__ q_abs, int qa_stride, const __nv_bfloat16* __restrict__ q,
                            int q_stride, int dn, __nv_bfloat16* __restrict__ out, int out_stride, float* __restrict__ part,
                            const __nv_bfloat16* __restrict__ cache, int num_pages, int page_size,
                            const int* __restrict__ block_table, int table_stride, const int* __restrict__ query_start_loc,
                            const int* __restrict__ seq_lens, int num_requests, const float* __restrict__ freq, int rot_dims,
                            const float* __restrict__ sinks, int H, int hb_log2, int rk, int dr, float scale_log2,
                            float rot_gain, int window) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ int s_req, s_tile;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr int kLmM = 16 * RG;
    const int rg = warp % RG, ch = warp / RG;              // row group of 16 rows; which half of the value columns
    const int qrow = lane >> 2, quad = lane & 3;
    const int D = rk + dr, LD = D + 8;                     // rows 16 bytes longer than D: ldmatrix hits every bank once
    const int HB = 1 << hb_log2, TM = kLmM >> hb_log2;
    const int splits = gridDim.z, split = blockIdx.z;

    if (tid == 0) {
        // The last CTAs of the grid take the first tiles: a request's late tokens see the most keys, and the tiles that
        // run longest should start first.  (A captured step's grid is an upper bound; the CTAs beyond the batch's own
        // tiles are then the FIRST to be scheduled, find no request and leave.)
        int t = gridDim.x - 1 - blockIdx.x, r = 0;
        for (; r < num_requests; ++r) {
            const int tiles = (query_start_loc[r + 1] - query_start_loc[r] + TM - 1) / TM;
            if (t < tiles) break;
            t -= tiles;
        }
        s_req = r;
        s_tile = t;
    }
    __syncthreads();
    const int r = s_req;
    if (r >= num_requests) return;
    const int q0 = query_start_loc[r];
    const int n = query_start_loc[r + 1] - q0;
    const int seq_len = seq_lens[r];
    const int tok0 = s_tile * TM;
    const int head0 = blockIdx.y * HB;
    const int* table = block_table + (size_t)r * table_stride;

    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* sK = sQ + (size_t)kLmM * LD;
    auto stage = [&](int s) { return sK + (size_t)s * kLmN * LD; };

    const int k_hi = seq_len - n + min(tok0 + TM, n);      // keys < k_hi are visible to the tile's last token
    const int tiles_all = (k_hi + kLmN - 1) / kLmN;
    // with a window the tile's first token sees nothing before its position - window + 1, and the later ones even less
    const int tile_lo = window > 0 ? max(0, seq_len - n + tok0 - window + 1) / kLmN : 0;
    const int per = (tiles_all - tile_lo + splits - 1) / splits;
    const int t_begin = tile_lo + split * per, t_end = min(tiles_all, t_begin + per);

    // A key row of a tile is copied by blockDim.x / 32 threads, 16 bytes at a time.  Its page number is looked up one
    // tile ahead (`page_of`), so that no copy waits for a block-table entry: with the lookup inside the copy loop every
    // 16-byte chunk stalled its thread for a trip to the L2, 8 us a tile.
    const int tpr = blockDim.x / kLmN;
    const int lrow = tid / tpr, lsub = tid % tpr;
    auto page_of = [&](int key0) {
        const int key = key0 + lrow;
        if (key >= k_hi) return -1;
        const int page = table[key / page_size];
        return (page >= 0 && page < num_pages) ? page : -1;
    };
    auto load_keys = [&](int s, int key0, int page) {
        const bool ok = page >= 0;
        const __nv_bfloat16* src = cache + ((size_t)(ok ? page : 0) * page_size + (ok ? (key0 + lrow) % page_size : 0)) * D;
        __nv_bfloat16* dst = stage(s) + lrow * LD;
        for (int chunk = lsub; chunk < D / 8; chunk += tpr) cp_async16(dst + chunk * 8, src + chunk * 8, ok);
    };

    // ---- query tile: [Uk^T q_plain (rk) | rot(q_rot) (dr)] per (token, head) row ----
    {
        const int chunks = rk / 8;
        for (int idx = tid; idx < kLmM * chunks; idx += blockDim.x) {
            const int row = idx / chunks, chunk = idx % chunks;
            const int tl = tok0 + (row >> hb_log2), head = head0 + (row & (HB - 1));
            const bool ok = tl < n && head < H;
            const __nv_bfloat16* src = q_abs + (size_t)(q0 + (ok ? tl : 0)) * qa_stride + (size_t)(ok ? head : 0) * rk + chunk * 8;
            cp_async16(sQ + row * LD + chunk * 8, src, ok);
        }
        const int pairs = dr / 2;
        for (int idx = tid; idx < kLmM * pairs; idx += blockDim.x) {
            const int row = idx / pairs, i = idx % pairs;
            const int tl = tok0 + (row >> hb_log2), head = head0 + (row & (HB - 1));
            float u = 0.f, v = 0.f;
            if (tl < n && head < H) {
                const __nv_bfloat16* src = q + (size_t)(q0 + tl) * q_stride + (size_t)head * (dn + dr) + dn + 2 * i;
                u = __bfloat162float(src[0]);
                v = __bfloat162float(src[1]);
                if (2 * i + 1 < rot_dims) {
                    float sn, cs;
                    sincosf((float)(seq_len - n + tl) * freq[i], &sn, &cs);
                    sn *= rot_gain;
                    cs *= rot_gain;
                    const float a = u * cs - v * sn, b = v * cs + u * sn;
                    u = a;
                    v = b;
                }
            }
            *reinterpret_cast<uint32_t*>(sQ + row * LD + rk + 2 * i) = pack_bf16(u, v);
        }
    }
    if (t_begin < t_end) load_keys(0, t_begin * kLmN, page_of(t_begin * kLmN));
    cp_async_commit();
    int page_next = t_begin + 1 < t_end ? page_of((t_begin + 1) * kLmN) : -1;

    int pos_row[2], head_row[2];
    bool row_ok[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = rg * 16 + qrow + 8 * h;
        const int tl = tok0 + (row >> hb_log2);
        head_row[h] = head0 + (row & (HB - 1));
        row_ok[h] = tl < n && head_row[h] < H;
        pos_row[h] = row_ok[h] ? seq_len - n + tl : -1;
    }
    const int warp_pos_min = seq_len - n + min(tok0 + ((rg * 16) >> hb_log2), n - 1);
    const int warp_pos_max = seq_len - n + min(tok0 + ((rg * 16 + 15) >> hb_log2), n - 1);

    float o[RKH / 8][4];
#pragma unroll
    for (int i = 0; i < RKH / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_run[2], l_run[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const bool with_sink = splits == 1 && sinks != nullptr && row_ok[h];
        m_run[h] = with_sink ? sinks[head_row[h]] * kLog2e : -INFINITY;
        l_run[h] = with_sink && quad == 0 ? 1.f : 0.f;
    }
    const int col_base = ch * RKH;                          // this warp's value columns: col_base .. col_base + RKH (< rk)
    const int mat = lane >> 3, rr = lane & 7;

    for (int t = t_begin; t < t_end; ++t) {
        const int key0 = t * kLmN;
        if (t + 1 < t_end) {
            load_keys((t + 1 - t_begin) & 1, key0 + kLmN, page_next);
            page_next = t + 2 < t_end ? page_of(key0 + 2 * kLmN) : -1;
        }
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const __nv_bfloat16* sKt = stage((t - t_begin) & 1);

        // ---- S = Q K^T : 16 x 32 per warp, over all rk + dr columns ----
        float s[kLmN / 8][4];
#pragma unroll
        for (int nt = 0; nt < kLmN / 8; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f; }
        {
            const int arow = rg * 16 + (mat & 1) * 8 + rr;
            const uint32_t a_base = smem_u32(sQ + arow * LD + (mat >> 1) * 8);
            const uint32_t b_base = smem_u32(sKt + ((mat >> 1) * 8 + rr) * LD + (mat & 1) * 8);
            // fragments of step kt + 1 are asked for before the products of step kt are issued: with two warps to a
            // scheduler nothing else hides the shared-memory latency
            const int ksteps = D / 16;
            uint32_t a0[4], a1[4], b0[kLmN / 16][4], b1[kLmN / 16][4];
            auto fetch = [&](uint32_t (&a)[4], uint32_t (&b)[kLmN / 16][4], int kt) {
                ldmatrix_x4(a, a_base + kt * 32);
#pragma unroll
                for (int np = 0; np < kLmN / 16; ++np) ldmatrix_x4(b[np], b_base + (np * 16 * LD + kt * 16) * 2);
            };
            auto multiply = [&](const uint32_t (&a)[4], const uint32_t (&b)[kLmN / 16][4]) {
#pragma unroll
                for (int np = 0; np < kLmN / 16; ++np) {
                    mma_bf16_16816(s[2 * np], a, b[np][0], b[np][1]);
                    mma_bf16_16816(s[2 * np + 1], a, b[np][2], b[np][3]);
                }
            };
            fetch(a0, b0, 0);
            int kt = 0;
            for (; kt + 1 < ksteps; kt += 2) {
                fetch(a1, b1, kt + 1);
                multiply(a0, b0);
                if (kt + 2 < ksteps) fetch(a0, b0, kt + 2);
                multiply(a1, b1);
            }
            if (kt < ksteps) multiply(a0, b0);
        }
        // ---- scale, causal mask where the tile touches the diagonal, running maximum ----
        const bool need_mask = key0 + kLmN - 1 > warp_pos_min || (window > 0 && key0 <= warp_pos_max - window);
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < kLmN / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int h = e >> 1;
                float v = s[nt][e] * scale_log2;
                if (need_mask) {
                    const int key = key0 + nt * 8 + quad * 2 + (e & 1);
                    v = (key <= pos_row[h] && (window <= 0 || key > pos_row[h] - window)) ? v : -INFINITY;
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
        for (int nt = 0; nt < kLmN / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float mref = m_run[e >> 1];
                const float p = (s[nt][e] == -INFINITY || mref == -INFINITY) ? 0.f : exp2f(s[nt][e] - mref);
                s[nt][e] = p;
                l_run[e >> 1] += p;
            }
        }
#pragma unroll
        for (int i = 0; i < RKH / 8; ++i) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
        // ---- O += P V, V = the tile's first rk columns ----
#pragma unroll
        for (int kp = 0; kp < kLmN / 16; ++kp) {
            uint32_t pf[4];
            pf[0] = pack_bf16(s[2 * kp][0], s[2 * kp][1]);
            pf[1] = pack_bf16(s[2 * kp][2], s[2 * kp][3]);
            pf[2] = pack_bf16(s[2 * kp + 1][0], s[2 * kp + 1][1]);
            pf[3] = pack_bf16(s[2 * kp + 1][2], s[2 * kp + 1][3]);
            const uint32_t v_base = smem_u32(sKt + (kp * 16 + (mat & 1) * 8 + rr) * LD + col_base + (mat >> 1) * 8);
#pragma unroll
            for (int nt = 0; nt < RKH / 16; ++nt) {
                if (col_base + nt * 16 < rk) {                 // uniform over the warp
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, v_base + nt * 32);
                    mma_bf16_16816(o[2 * nt], pf, b[0], b[1]);
                    mma_bf16_16816(o[2 * nt + 1], pf, b[2], b[3]);
                }
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();

#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float l = l_run[h];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        if (!row_ok[h]) continue;
        const int row = rg * 16 + qrow + 8 * h;
        const int token = q0 + tok0 + (row >> hb_log2);
        if (splits == 1) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16* dst = out + (size_t)token * out_stride + (size_t)head_row[h] * rk;
#pragma unroll
            for (int i = 0; i < RKH / 8; ++i) {
                const int col = col_base + i * 8 + quad * 2;
                if (col < rk)
                    *reinterpret_cast<uint32_t*>(dst + col) = pack_bf16(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
            }
        } else {
            float* dst = part + (((size_t)token * H + head_row[h]) * splits + split) * (rk + 2);
            if (ch == 0 && quad == 0) {
                dst[0] = m_run[h];
                dst[1] = l;
            }
#pragma unroll
            for (int i = 0; i < RKH / 8; ++i) {
                const int col = col_base + i * 8 + quad * 2;
                if (col < rk) {
                    dst[2 + col] = o[i][2 * h];
                    dst[3 + col] = o[i][2 * h + 1];
                }
            }
        }
    }
}

// Merge the splits of a (token, head): M = max(sink, m_s), L = 2^(sink - M) + sum l_s 2^(m_s - M),
// out = sum acc_s 2^(m_s - M) / L.  A block per (token, head), a thread per column.
__global__ void latent_attention_merge_kernel(const float* __restrict__ part, const float* __restrict__ sinks,
                                              __nv_bfloat16* __restrict__ out, int out_stride, int H, int rk, int splits,
                                              int rows) {
    const int w = blockIdx.x, lane = threadIdx.x;
    if (w >= rows) return;
    const int token = w / H, head = w % H;
    const float* p = part + (size_t)w * splits * (rk + 2);
    const float sink = sinks ? sinks[head] * kLog2e : -INFINITY;
    float M = sink;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, p[(size_t)s * (rk + 2)]);
    float L = sink == -INFINITY ? 0.f : exp2f(sink - M);
    for (int s = 0; s < splits; ++s) {
        const float m = p[(size_t)s * (rk + 2)];
        if (m != -INFINITY) L += p[(size_t)s * (rk + 2) + 1] * exp2f(m - M);
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    for (int c = lane; c < rk; c += blockDim.x) {
        float acc = 0.f;
#pragma unroll 4
        for (int s = 0; s < splits; ++s) {
            const float m = p[(size_t)s * (rk + 2)];
            if (m != -INFINITY) acc += p[(size_t)s * (rk + 2) + 2 + c] * exp2f(m - M);
        }
        out[(size_t)token * out_stride + (size_t)head * rk + c] = __float2bfloat16_rn(acc * inv);
    }
}

template <int RKH, int CS, int RG>
static int launch_latent_mma(dim3 grid, size_t smem, cudaStream_t stream, const void* q_abs, int qa_stride, const void* q,
                             int q_stride, int dn, void* out, int out_stride, float* part, const void* cache, int num_pages,
                             int page_size, const int* bt, int ts, const int* qsl, const int* sl, int R, const float* freq,
                             int rot_dims, const float* sinks, int H, int hb_log2, int rk, int dr, float scale_log2,
                             float rot_gain, int window) {
    static SmemLimit limit;
    auto kernel = latent_attention_mma_kernel<RKH, CS, RG>;
    if (smem > 48 * 1024 && raise_smem_limit(limit, kernel, 200 * 1024, "latent_attention_mma") != 0) return -2;
    kernel<<<grid, 32 * RG * CS, smem, stream>>>((const __nv_bfloat16*)q_abs, qa_stride, (const __nv_bfloat16*)q, q_stride, dn,
                                             (__nv_bfloat16*)out, out_stride, part, (const __nv_bfloat16*)cache, num_pages,
                                             page_size, bt, ts, qsl, sl, R, freq, rot_dims, sinks, H, hb_log2, rk, dr,
                                             scale_log2, rot_gain, window);
    return 0;
}

}  // namespace cib

using namespace cib;

extern "C" int cib_latent_attention_mma_supports(int rk, int dr, int dn) {
    return rk > 0 && rk % 16 == 0 && rk <= 512 && dr >= 0 && dr % 16 == 0 && dn >= 0;
}

// Heads side by side in a query tile of `rows` rows: the smallest power of two that holds min(H, rows) heads.
static int head_block_log2(int H, int rows) {
    int k = 0;
    while ((1 << k) < H && (1 << k) < rows) ++k;
    return k;
}

// Row tiles a launch needs for requests of these numbers of new tokens, with query tiles of `rows` (64 or 32) rows.
extern "C" int cib_latent_attention_mma_tiles(const int* query_lens, int num_requests, int H, int rows) {
    const int tm = rows >> head_block_log2(H, rows);
    long long tiles = 0;
    for (int i = 0; i < num_requests; ++i) tiles += (query_lens[i] + tm - 1) / tm;
    return (int)(tiles > 0x7fffffff ? 0x7fffffff : tiles);
}

// `scratch`: splits > 1 needs num_tokens * H * splits * (rk + 2) floats.  `sinks` 32-bit or null.
extern "C" int cib_latent_attention_mma(const void* q_abs, int qa_stride, const void* q, int q_stride, int dn, void* out,
                                        int out_stride, float* scratch, const void* cache, int num_pages, int page_size,
                                        const int* block_table, int table_stride, const int* query_start_loc,
                                        const int* seq_lens, int num_requests, int row_tiles, int tile_rows, const float* freq,
                                        int rot_dims, const float* sinks, int num_tokens, int H, int rk, int dr, float scale,
                                        int splits, float rot_gain, int window, cudaStream_t stream) {
    CIB_REQUIRE(cib_latent_attention_mma_supports(rk, dr, dn), "latent_attention_mma: sizes rk=%d dr=%d are not taken", rk, dr);
    CIB_REQUIRE(num_tokens >= 0 && H > 0 && num_requests > 0 && row_tiles >= 0, "latent_attention_mma: bad sizes");
    CIB_REQUIRE(page_size > 0 && num_pages > 0 && table_stride > 0, "latent_attention_mma: bad cache geometry");
    CIB_REQUIRE(rot_dims >= 0 && rot_dims <= dr && rot_dims % 2 == 0 && (rot_dims == 0 || freq), "latent_attention_mma: bad rotary part");
    CIB_REQUIRE(qa_stride % 8 == 0 && out_stride % 2 == 0, "latent_attention_mma: rows must start on 16-byte boundaries");
    CIB_REQUIRE(splits >= 1 && splits <= 65535 && (splits == 1 || scratch != nullptr), "latent_attention_mma: bad split");
    CIB_REQUIRE(tile_rows == 64 || tile_rows == 32, "latent_attention_mma: query tiles have 64 or 32 rows");
    CIB_REQUIRE(window >= 0, "latent_attention_mma: window must be >= 0 (0 = all keys)");
    if (num_tokens == 0 || row_tiles == 0) return 0;
    const int hb_log2 = head_block_log2(H, tile_rows);
    dim3 grid(row_tiles, (H + (1 << hb_log2) - 1) >> hb_log2, splits);
    const int D = rk + dr;
    const size_t smem = (size_t)(tile_rows + 2 * kLmN) * (D + 8) * sizeof(__nv_bfloat16);
    const float scale_log2 = scale * kLog2e;
    int rc;
#define CIB_LM_ARGS                                                                                                        \
    grid, smem, stream, q_abs, qa_stride, q, q_stride, dn, out, out_stride, scratch, cache, num_pages, page_size, block_table, \
        table_stride, query_start_loc, seq_lens, num_requests, freq, rot_dims, sinks, H, hb_log2, rk, dr, scale_log2, \
        rot_gain, window
#define CIB_LM_GO(RKH, CS) \
    rc = tile_rows == 64 ? launch_latent_mma<RKH, CS, 4>(CIB_LM_ARGS) : launch_latent_mma<RKH, CS, 2>(CIB_LM_ARGS)
    if (rk <= 32) CIB_LM_GO(32, 1);
    else if (rk <= 64) CIB_LM_GO(64, 1);
    else if (rk <= 128) CIB_LM_GO(128, 1);
    else if (rk <= 256) CIB_LM_GO(256, 1);
    else CIB_LM_GO(256, 2);
#undef CIB_LM_GO
#undef CIB_LM_ARGS
    if (rc != 0) return rc;
    CIB_LAUNCH_CHECK("latent_attention_mma");
    if (splits > 1) {
        const int rows = num_tokens * H;
        latent_attention_merge_kernel<<<rows, rk >= 256 ? 256 : 128, 0, stream>>>(scratch, sinks, (__nv_bfloat16*)out, out_stride, H, rk,
                                                                           splits, rows);
        CIB_LAUNCH_CHECK("latent_attention_merge");
    }
    return 0;
}

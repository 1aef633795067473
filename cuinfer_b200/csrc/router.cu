// Choice of experts by a router.  A warp per token; everything 32-bit.
//  * router_topk: from logits z[t, 0..E-1] the `top` largest (the lower index wins a tie) and their weights, the softmax
//    over the chosen logits only.
//  * router_scored_topk: scores s = sigmoid(z); the choice goes by s + correction[e] (a learned number per expert, may be
//    null), the weights by s alone, times `scale`, not renormalised.  The experts form `groups` equal groups of
//    neighbours; a group's mark is the sum of its two largest choice scores (of its one, for groups of one), and only
//    experts of the `keep` groups with the largest marks can be chosen (the lower group wins a tie).
#include "common.cuh"

namespace cib {

constexpr int kRouterWarps = 8;
constexpr int kRouterPerLane = 32;           // up to 1024 experts

__global__ void __launch_bounds__(kRouterWarps * 32)
router_topk_kernel(const float* __restrict__ logits, int stride, int experts, int top, int* __restrict__ choice,
                   float* __restrict__ weight, int num_tokens) {
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * kRouterWarps + (threadIdx.x >> 5);
    if (t >= num_tokens) return;
    float z[kRouterPerLane];
#pragma unroll
    for (int c = 0; c < kRouterPerLane; ++c) {
        const int e = c * 32 + lane;
        z[c] = e < experts ? logits[(size_t)t * stride + e] : -INFINITY;
        if (z[c] != z[c]) z[c] = -INFINITY;               // a NaN logit is never chosen
    }
    float first = 0.f, sum = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = 0x7fffffff;
#pragma unroll
        for (int c = 0; c < kRouterPerLane; ++c) {
            const int e = c * 32 + lane;
            if (e < experts && (z[c] > best || (z[c] == best && e < at))) { best = z[c]; at = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at == 0x7fffffff) at = -1;
        if (k == 0) first = best;
        const float p = at >= 0 ? expf(best - first) : 0.f;
        sum += p;
        if (lane == 0) {
            choice[(size_t)t * top + k] = at;
            weight[(size_t)t * top + k] = p;
        }
#pragma unroll
        for (int c = 0; c < kRouterPerLane; ++c)
            if (c * 32 + lane == at) z[c] = -INFINITY;
    }
    __syncwarp();
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
    for (int k = lane; k < top; k += 32) weight[(size_t)t * top + k] *= inv;
}

constexpr int kScoredWarps = 4;

// Shared memory per warp: E choice scores, then `groups` marks.
__global__ void __launch_bounds__(kScoredWarps * 32)
router_scored_topk_kernel(const float* __restrict__ logits, int stride, int experts, int top, const float* __restrict__ correction,
                          int groups, int keep, float scale, int* __restrict__ choice, float* __restrict__ weight,
                          int num_tokens) {
    extern __shared__ float scored_s[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * kScoredWarps + warp;
    if (t >= num_tokens) return;                                  // a whole warp leaves; nothing below syncs the block
    float* cs = scored_s + (size_t)warp * (experts + groups);
    float* mark = cs + experts;
    const float* z = logits + (size_t)t * stride;
    for (int e = lane; e < experts; e += 32) {
        const float s = 1.f / (1.f + expf(-z[e]));
        float c = s + (correction ? correction[e] : 0.f);
        if (c != c) c = -INFINITY;                                // a NaN is never chosen
        cs[e] = c;
    }
    __syncwarp();
    if (groups > 1) {
        const int size = experts / groups;
        for (int g = lane; g < groups; g += 32) {
            float a = -INFINITY, b = -INFINITY;                   // the two largest of the group
            for (int i = 0; i < size; ++i) {
                const float c = cs[g * size + i];
                if (c > a) { b = a; a = c; }
                else if (c > b) b = c;
            }
            mark[g] = size > 1 ? a + b : a;
        }
        __syncwarp();
        // the `keep` best groups stay; a kept group is marked with +infinity so that it is not taken twice
        for (int k = 0; k < keep; ++k) {
            float best = -INFINITY;
            int at = 0x7fffffff;
            for (int g = lane; g < groups; g += 32) {
                const float m = mark[g];
                if (m != INFINITY && (at == 0x7fffffff || m > best)) { best = m; at = g; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (oa != 0x7fffffff && (at == 0x7fffffff || ob > best || (ob == best && oa < at))) { best = ob; at = oa; }
            }
            if (at != 0x7fffffff && lane == 0) mark[at] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < experts; e += 32)
            if (mark[e / size] != INFINITY) cs[e] = -INFINITY;
        __syncwarp();
    }
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            const float c = cs[e];
            if (c > best) { best = c; at = e; }                   // a lane walks upwards: the lower index keeps a tie
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at == 0x7fffffff) at = -1;
        if (lane == 0) {
            choice[(size_t)t * top + k] = at;
            weight[(size_t)t * top + k] = at >= 0 ? scale / (1.f + expf(-z[at])) : 0.f;
            if (at >= 0) cs[at] = -INFINITY;
        }
        __syncwarp();
    }
}

}  // namespace cib

extern "C" int cib_router_scored_topk(const float* logits, int stride, int experts, int top, const float* correction,
                                      int groups, int keep, float scale, int* choice, float* weight, int num_tokens,
                                      cudaStream_t stream) {
    using namespace cib;
    CIB_REQUIRE(experts > 0 && top > 0 && top <= experts, "router_scored_topk: top %d of %d experts", top, experts);
    CIB_REQUIRE(groups > 0 && experts % groups == 0 && keep > 0 && keep <= groups, "router_scored_topk: %d groups (%d kept) of %d experts", groups, keep, experts);
    CIB_REQUIRE((long long)keep * (experts / groups) >= top, "router_scored_topk: %d kept groups of %d experts cannot give %d", keep, experts / groups, top);
    CIB_REQUIRE(experts + groups <= 8192, "router_scored_topk: %d experts are beyond this kernel", experts);
    if (num_tokens == 0) return 0;
    const size_t smem = (size_t)kScoredWarps * (experts + groups) * sizeof(float);
    static SmemLimit limit;
    if (smem > 48 * 1024 && raise_smem_limit(limit, router_scored_topk_kernel, 200 * 1024, "router_scored_topk") != 0) return -2;
    router_scored_topk_kernel<<<(num_tokens + kScoredWarps - 1) / kScoredWarps, kScoredWarps * 32, smem, stream>>>(
        logits, stride, experts, top, correction, groups, keep, scale, choice, weight, num_tokens);
    CIB_LAUNCH_CHECK("router_scored_topk");
    return 0;
}

extern "C" int cib_router_topk(const float* logits, int stride, int experts, int top, int* choice, float* weight,
                               int num_tokens, cudaStream_t stream) {
    using namespace cib;
    CIB_REQUIRE(experts > 0 && top > 0 && top <= experts, "router_topk: top %d of %d experts", top, experts);
    CIB_REQUIRE(experts <= 32 * kRouterPerLane, "router_topk: %d experts are beyond %d", experts, 32 * kRouterPerLane);
    if (num_tokens == 0) return 0;
    router_topk_kernel<<<(num_tokens + kRouterWarps - 1) / kRouterWarps, kRouterWarps * 32, 0, stream>>>(logits, stride, experts, top, choice, weight, num_tokens);
    CIB_LAUNCH_CHECK("router_topk");
    return 0;
}

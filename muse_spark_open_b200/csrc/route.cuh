// Expert choice of one token by one warp: softmax -> top-k -> renormalise over the chosen (the benchmark's
// routing rule; the renormalisation is the one of muse_moe_w4a16/reference.py:82).  Shared by the router kernel
// and the experts' GEMM.
#pragma once
#include <cstdint>

#include "ptx.cuh"

namespace msk {

// order-preserving map float -> uint32 (larger float <=> larger integer)
__device__ __forceinline__ uint32_t float_ordered(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float ordered_float(uint32_t o) {
    return __uint_as_float((o & 0x80000000u) ? (o & 0x7fffffffu) : ~o);
}

// logits[0..n), n <= 32 * NV.  Lanes 0..top_k-1 write ids[lane] (global expert id) and wts[lane] (probability,
// renormalised over the chosen).  Ties go to the lower expert id.  Two warp reductions per choice.
template <int NV>
__device__ __forceinline__ void route_token_nv(const float* logits, int n, int top_k, int lane, int* ids, float* wts) {
    uint32_t v[NV];
    uint32_t mxo = 0;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int e = lane + 32 * i;
        v[i] = e < n ? float_ordered(__ldcg(logits + e)) : 0u;
        mxo = max(mxo, v[i]);
    }
    const float mx = ordered_float(__reduce_max_sync(0xffffffffu, mxo));
    float sum = 0.0f, my_p = 0.0f;
    int my_id = 0;
    for (int k = 0; k < top_k; ++k) {
        uint32_t best = 0;
#pragma unroll
        for (int i = 0; i < NV; ++i) best = max(best, v[i]);
        best = __reduce_max_sync(0xffffffffu, best);
        int cand = 0x7fffffff;  // this lane's lowest expert id holding the maximum
#pragma unroll
        for (int i = NV - 1; i >= 0; --i)
            if (v[i] == best) cand = lane + 32 * i;
        const int bi = __reduce_min_sync(0xffffffffu, cand);
        const float pk = __expf(ordered_float(best) - mx);
        sum += pk;
        if (lane == k) my_id = bi, my_p = pk;
#pragma unroll
        for (int i = 0; i < NV; ++i)
            if (lane + 32 * i == bi) v[i] = 0u;
    }
    if (lane < top_k) {
        ids[lane] = my_id;
        wts[lane] = my_p / sum;
    }
}
// The reference layer's own rule (muse_decode_layer/reference.py:419-424,462-463): scores = sigmoid(multiplier *
// logit); the top-k of score + bias are chosen (ties to the lower expert id); the weights are the UNBIASED scores
// of the chosen, divided by their sum + 1e-15.
template <int NV>
__device__ __forceinline__ void route_token_sigmoid_nv(const float* logits, const float* bias, float multiplier, int n,
                                                       int top_k, int lane, int* ids, float* wts) {
    uint32_t key[NV];
    float sc[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int e = lane + 32 * i;
        sc[i] = 0.0f, key[i] = 0u;
        if (e < n) {
            sc[i] = 1.0f / (1.0f + expf(-multiplier * __ldcg(logits + e)));
            key[i] = float_ordered(sc[i] + (bias != nullptr ? bias[e] : 0.0f));
        }
    }
    float sum = 0.0f, my_p = 0.0f;
    int my_id = 0;
    for (int k = 0; k < top_k; ++k) {
        uint32_t best = 0;
#pragma unroll
        for (int i = 0; i < NV; ++i) best = max(best, key[i]);
        best = __reduce_max_sync(0xffffffffu, best);
        int cand = 0x7fffffff;
        float cand_s = 0.0f;
#pragma unroll
        for (int i = NV - 1; i >= 0; --i)
            if (key[i] == best) cand = lane + 32 * i, cand_s = sc[i];
        const int bi = __reduce_min_sync(0xffffffffu, cand);
        const float pk = __shfl_sync(0xffffffffu, cand_s, bi & 31);  // the lane that holds expert bi
        sum += pk;
        if (lane == k) my_id = bi, my_p = pk;
#pragma unroll
        for (int i = 0; i < NV; ++i)
            if (lane + 32 * i == bi) key[i] = 0u;
    }
    if (lane < top_k) {
        ids[lane] = my_id;
        wts[lane] = my_p / (sum + 1e-15f);
    }
}
__device__ __forceinline__ void route_token_sigmoid(const float* logits, const float* bias, float multiplier, int n, int top_k,
                                                    int lane, int* ids, float* wts) {
    if (n <= 128) route_token_sigmoid_nv<4>(logits, bias, multiplier, n, top_k, lane, ids, wts);
    else route_token_sigmoid_nv<8>(logits, bias, multiplier, n, top_k, lane, ids, wts);
}

__device__ __forceinline__ void route_token(const float* logits, int n, int top_k, int lane, int* ids, float* wts) {
    if (n <= 128) route_token_nv<4>(logits, n, top_k, lane, ids, wts);
    else route_token_nv<8>(logits, n, top_k, lane, ids, wts);
}

}  // namespace msk

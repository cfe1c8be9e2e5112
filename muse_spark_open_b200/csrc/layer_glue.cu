// The small kernels between the big ones of the decoder layer, and the layer's launch chain.
//   prep_norm    x = bf16(rmsnorm(stream) * (1 + w)), one block per token (the rounding point of the
//                reference); also leaves ssq[t] = sum stream^2.
//   router       FP32 logits[t, e] = rs[t] * sum_k (stream1[t,k] * (1 + w[k])) * R[e, k] + bias[e] on
//                CUDA cores (expert ids must not depend on tensor-core rounding).  Blocks of 32 tokens x 32
//                experts x 128 of K; the last block of a (token group, expert tile) to finish (ticket) adds
//                the H/128 partials in a fixed order, so ids are reproducible.
#include "msk.h"
#include "ptx.cuh"
#include "route.cuh"

namespace msk {

__global__ void __launch_bounds__(256) prep_norm_kernel(const float* __restrict__ stream, const __nv_bfloat16* __restrict__ w,
                                                        __nv_bfloat16* __restrict__ xn, float* __restrict__ ssq, int H,
                                                        float eps) {
    __shared__ float red[8];
    __shared__ float rs_s;
    const int t = blockIdx.x, tid = threadIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    constexpr int kMaxVec = 8;  // H <= 8192
    float4 v[kMaxVec];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
        const int d = tid * 4 + i * 1024;
        v[i] = make_float4(0, 0, 0, 0);
        if (d < H) v[i] = __ldcg(reinterpret_cast<const float4*>(stream + static_cast<size_t>(t) * H + d));
        ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    }
    ss = warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    if (tid == 0) {
        const float tot = ((red[0] + red[1]) + (red[2] + red[3])) + ((red[4] + red[5]) + (red[6] + red[7]));
        ssq[t] = tot;
        rs_s = 1.0f / sqrtf(tot / H + eps);
    }
    __syncthreads();
    const float rs = rs_s;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
        const int d = tid * 4 + i * 1024;
        if (d < H) {
            const uint2 pw = *reinterpret_cast<const uint2*>(w + d);
            *reinterpret_cast<uint2*>(xn + static_cast<size_t>(t) * H + d) =
                make_uint2(pack_bf16(v[i].x * rs * (1.0f + bf16lo(pw.x)), v[i].y * rs * (1.0f + bf16hi(pw.x))),
                           pack_bf16(v[i].z * rs * (1.0f + bf16lo(pw.y)), v[i].w * rs * (1.0f + bf16hi(pw.y))));
        }
    }
}

struct RouterArgs {
    const float* s1;        // [T, H]
    const __nv_bfloat16* w; // [H]
    float* ssq;             // [parts + 1, T]; the last row receives the totals
    int ssq_parts;
    float eps;
    const float* R;         // [E, H]
    const float* bias;      // [E] or null
    float* part;            // [KS, T, E]
    int* ticket;            // [token groups x expert tiles] then [token groups]
    int top_k;
    int* ids_out;           // [T, top_k]
    float* wts_out;
    float* logits;          // [T, E]
    int T, H, E;
    int sigmoid_bias;       // 0: softmax over logits + bias; 1: sigmoid(multiplier * logit), chosen by score + bias
    float multiplier;
    int phases;             // 128-k tiles a block walks: H = gridDim.x * phases * 128
};

constexpr int kRouterK = 128;   // k per block (one load phase)
constexpr int kRouterT = 32;    // tokens per block
constexpr int kRouterE = 32;    // experts per block

__global__ void __launch_bounds__(256) router_kernel(RouterArgs p) {
    __shared__ __align__(16) float Rs[kRouterE][kRouterK + 4];  // row stride 132 floats: 16-byte rows, no bank conflicts
    __shared__ __align__(16) float hs[kRouterT][kRouterK];
    __shared__ int last;
    const int ks = blockIdx.x, et = blockIdx.y, tid = threadIdx.x;
    const int KS = gridDim.x;  // K splits = H / (128 * phases)
    const int e0 = et * kRouterE, kb = ks * kRouterK * p.phases;
    const int ne = min(kRouterE, p.E - e0), n_tg = (p.T + kRouterT - 1) / kRouterT;
    const int tw = tid >> 5, el = tid & 31;  // warp w owns tokens w, w+8, w+16, w+24; lane = expert
    // both tiles are 32 rows x 32 float4; thread -> rows tw, tw+8, tw+16, tw+24, float4 column el.  All four loads
    // are issued before the first use; rows past the end re-read the last valid row and are zeroed.
    // the first tile of router weights does not depend on the previous kernel: requested before the wait
    auto load_r = [&](int k0, float4 (&r)[4]) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
            r[j] = __ldg(reinterpret_cast<const float4*>(p.R + static_cast<size_t>(e0 + min(tw + 8 * j, ne - 1)) * p.H + k0) + el);
    };
    float4 r_first[4];
    load_r(kb, r_first);
    pdl_wait();
    pdl_launch_dependents();
    // With many token groups a block walks `phases` tiles of 128 k: fewer, longer blocks (the grid stays within one
    // wave of CTAs) and fewer partials for the chain of global round trips at the end.
    for (int tg = blockIdx.z; tg < n_tg; tg += gridDim.z) {
    const int t0 = tg * kRouterT, nt = min(kRouterT, p.T - t0);
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int ph = 0; ph < p.phases; ++ph) {
        const int k0 = kb + ph * kRouterK;
        float4 r[4], h[4];
        if (ph == 0) {
#pragma unroll
            for (int j = 0; j < 4; ++j) r[j] = r_first[j];
        } else {
            load_r(k0, r);
        }
        const uint2 wraw = __ldg(reinterpret_cast<const uint2*>(p.w + k0) + el);
#pragma unroll
        for (int j = 0; j < 4; ++j)
            h[j] = __ldcg(reinterpret_cast<const float4*>(p.s1 + static_cast<size_t>(t0 + min(tw + 8 * j, nt - 1)) * p.H + k0) + el);
        const float w0 = 1.0f + bf16lo(wraw.x), w1 = 1.0f + bf16hi(wraw.x), w2 = 1.0f + bf16lo(wraw.y), w3 = 1.0f + bf16hi(wraw.y);
        __syncthreads();  // the previous tile's (or group's) use of Rs, hs and `last` is over
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            *reinterpret_cast<float4*>(&Rs[tw + 8 * j][4 * el]) = tw + 8 * j < ne ? r[j] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            *reinterpret_cast<float4*>(&hs[tw + 8 * j][4 * el]) =
                tw + 8 * j < nt ? make_float4(h[j].x * w0, h[j].y * w1, h[j].z * w2, h[j].w * w3) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
        __syncthreads();
#pragma unroll 8
        for (int k4 = 0; k4 < kRouterK / 4; ++k4) {
            const float4 rr = *reinterpret_cast<const float4*>(&Rs[el][4 * k4]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (tw + 8 * j >= nt) break;  // warp-uniform
                const float4 hh = *reinterpret_cast<const float4*>(&hs[tw + 8 * j][4 * k4]);
                acc[j] = fmaf(hh.x, rr.x, acc[j]), acc[j] = fmaf(hh.y, rr.y, acc[j]);
                acc[j] = fmaf(hh.z, rr.z, acc[j]), acc[j] = fmaf(hh.w, rr.w, acc[j]);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int t = tw + 8 * j;
        if (t < nt && el < ne) p.part[(static_cast<size_t>(ks) * p.T + t0 + t) * p.E + e0 + el] = acc[j];
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) last = atomicAdd(p.ticket + tg * gridDim.y + et, 1) == KS - 1;
    __syncthreads();
    if (!last) continue;
    __threadfence();
    // per-token 1/rms: lane q sums parts q, q + 32, ...; all four tokens' loads are in flight together
    float* rs_s = &hs[0][0];
    {
        float ss[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int q = el; q < p.ssq_parts; q += 32)
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (tw + 8 * j < nt) ss[j] += __ldcg(p.ssq + q * p.T + t0 + tw + 8 * j);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss[j] += __shfl_xor_sync(0xffffffffu, ss[j], o);
            if (el == 0 && tw + 8 * j < nt) {
                rs_s[tw + 8 * j] = rsqrtf(ss[j] / p.H + p.eps);
                if (et == 0) p.ssq[p.ssq_parts * p.T + t0 + tw + 8 * j] = ss[j];  // total, one value for the experts' GEMM
            }
        }
    }
    float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int s0 = 0; s0 < KS; s0 += 8) {  // KS is a multiple of 8; 32 loads in flight
        float v[4][8];
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int i = 0; i < 8; ++i)
                v[j][i] = (tw + 8 * j < nt && el < ne)
                              ? __ldcg(p.part + (static_cast<size_t>(s0 + i) * p.T + t0 + tw + 8 * j) * p.E + e0 + el)
                              : 0.0f;
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int i = 0; i < 8; ++i) sum[j] += v[j][i];
    }
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int t = tw + 8 * j;
        if (t < nt && el < ne) {
            float o = sum[j] * rs_s[t];
            if (p.bias != nullptr && !p.sigmoid_bias) o += p.bias[e0 + el];
            p.logits[static_cast<size_t>(t0 + t) * p.E + e0 + el] = o;
        }
    }
    if (tid == 0) p.ticket[tg * gridDim.y + et] = 0;  // ready for the next call
    // the last expert tile of this token group chooses the experts: a warp per token, 4 tokens per warp
    __threadfence();
    __syncthreads();
    int* ticket2 = p.ticket + n_tg * gridDim.y + tg;
    if (tid == 0) last = atomicAdd(ticket2, 1) == static_cast<int>(gridDim.y) - 1;
    __syncthreads();
    if (!last) continue;
    __threadfence();
    for (int j = 0; j < 4; ++j) {
        const int t = tw + 8 * j;
        if (t < nt) {
            if (p.sigmoid_bias)
                route_token_sigmoid(p.logits + static_cast<size_t>(t0 + t) * p.E, p.bias, p.multiplier, p.E, p.top_k, el,
                                    p.ids_out + (t0 + t) * p.top_k, p.wts_out + (t0 + t) * p.top_k);
            else
                route_token(p.logits + static_cast<size_t>(t0 + t) * p.E, p.E, p.top_k, el, p.ids_out + (t0 + t) * p.top_k,
                            p.wts_out + (t0 + t) * p.top_k);
        }
    }
    if (tid == 0) *ticket2 = 0;
    }
}

// Many tokens: one block takes 32 tokens x all experts (<= 128) x `phases` tiles of 128 k.  Thread = 4 tokens x 4
// experts (16 FP32 accumulators: 8 shared-memory loads per 64 FMAs, where the kernel above has 5 per 16), the grid is
// about one block per SM, and there is one ticket per token group instead of two stages: the block that draws the
// last ticket adds the K splits' partials in split order, writes the logits and chooses the experts.  A thread ends
// up with the logits of tokens tw + 8 i and experts lane + 32 j: exactly what a warp needs to choose for its tokens.
constexpr int kWideE = 128;
constexpr int kRouterWideSmem = (kWideE * (kRouterK + 4) + kRouterT * kRouterK) * 4;

__global__ void __launch_bounds__(256) router_wide_kernel(RouterArgs p) {
    extern __shared__ __align__(16) float wsm[];
    float (*Rs)[kRouterK + 4] = reinterpret_cast<float (*)[kRouterK + 4]>(wsm);                     // [128][132]
    float (*hs)[kRouterK] = reinterpret_cast<float (*)[kRouterK]>(wsm + kWideE * (kRouterK + 4));  // [32][128]
    __shared__ int last;
    const int ks = blockIdx.x, tg = blockIdx.y, tid = threadIdx.x, KS = gridDim.x;
    const int tw = tid >> 5, el = tid & 31;
    const int kb = ks * kRouterK * p.phases;
    const int t0 = tg * kRouterT, nt = min(kRouterT, p.T - t0);
    auto load_r = [&](int k0, float4 (&r)[16]) {  // rows tw + 8 j of the weight tile, float4 column el
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int e = tw + 8 * j;
            r[j] = e < p.E ? __ldg(reinterpret_cast<const float4*>(p.R + static_cast<size_t>(e) * p.H + k0) + el)
                           : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
    };
    float4 r[16];
    load_r(kb, r);  // the router weights do not depend on the previous kernel
    pdl_wait();
    pdl_launch_dependents();
    float acc[4][4];  // [token tw + 8 i][expert el + 32 j]
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    uint2 wraw = make_uint2(0, 0);
    float4 h[4];
    auto load_h = [&](int k0) {
        wraw = __ldg(reinterpret_cast<const uint2*>(p.w + k0) + el);
#pragma unroll
        for (int i = 0; i < 4; ++i)
            h[i] = __ldcg(reinterpret_cast<const float4*>(p.s1 + static_cast<size_t>(t0 + min(tw + 8 * i, nt - 1)) * p.H + k0) + el);
    };
    load_h(kb);
    for (int ph = 0; ph < p.phases; ++ph) {
        const float w0 = 1.0f + bf16lo(wraw.x), w1 = 1.0f + bf16hi(wraw.x), w2 = 1.0f + bf16lo(wraw.y), w3 = 1.0f + bf16hi(wraw.y);
        __syncthreads();  // the previous tile has been used
#pragma unroll
        for (int j = 0; j < 16; ++j) *reinterpret_cast<float4*>(&Rs[tw + 8 * j][4 * el]) = r[j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
            *reinterpret_cast<float4*>(&hs[tw + 8 * i][4 * el]) =
                tw + 8 * i < nt ? make_float4(h[i].x * w0, h[i].y * w1, h[i].z * w2, h[i].w * w3) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        __syncthreads();
        if (ph + 1 < p.phases) {  // the next tile's loads fly under this tile's arithmetic
            load_r(kb + (ph + 1) * kRouterK, r);
            load_h(kb + (ph + 1) * kRouterK);
        }
#pragma unroll 4
        for (int k4 = 0; k4 < kRouterK / 4; ++k4) {
            float4 rr[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) rr[j] = *reinterpret_cast<const float4*>(&Rs[el + 32 * j][4 * k4]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 hh = *reinterpret_cast<const float4*>(&hs[tw + 8 * i][4 * k4]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(hh.x, rr[j].x, acc[i][j]), acc[i][j] = fmaf(hh.y, rr[j].y, acc[i][j]);
                    acc[i][j] = fmaf(hh.z, rr[j].z, acc[i][j]), acc[i][j] = fmaf(hh.w, rr[j].w, acc[i][j]);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int t = tw + 8 * i;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (t < nt && el + 32 * j < p.E) p.part[(static_cast<size_t>(ks) * p.T + t0 + t) * p.E + el + 32 * j] = acc[i][j];
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) last = atomicAdd(p.ticket + tg, 1) == KS - 1;
    __syncthreads();
    if (!last) return;
    __threadfence();
    // per-token 1/rms: lane q sums parts q, q + 32, ...
    float rs[4];
    {
        float ss[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int q = el; q < p.ssq_parts; q += 32)
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (tw + 8 * i < nt) ss[i] += __ldcg(p.ssq + q * p.T + t0 + tw + 8 * i);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss[i] += __shfl_xor_sync(0xffffffffu, ss[i], o);
            rs[i] = rsqrtf(ss[i] / p.H + p.eps);
            if (el == 0 && tw + 8 * i < nt) p.ssq[p.ssq_parts * p.T + t0 + tw + 8 * i] = ss[i];  // total, one value for the experts' GEMM
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    // split order (the sum does not depend on which block came last), four splits' loads in flight together: one
    // round trip to L2 per batch, not per split
    for (int s0 = 0; s0 < KS; s0 += 4) {
        float v[4][4][4];
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    v[q][i][j] = (s0 + q < KS && tw + 8 * i < nt && el + 32 * j < p.E)
                                     ? __ldcg(p.part + (static_cast<size_t>(s0 + q) * p.T + t0 + tw + 8 * i) * p.E + el + 32 * j)
                                     : 0.0f;
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] += v[q][i][j];
    }
    for (int i = 0; i < 4; ++i) {
        const int t = tw + 8 * i;
        if (t >= nt) break;  // warp-uniform
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int e = el + 32 * j;
            if (e < p.E) {
                float o = acc[i][j] * rs[i];
                if (p.bias != nullptr && !p.sigmoid_bias) o += p.bias[e];
                p.logits[static_cast<size_t>(t0 + t) * p.E + e] = o;
            }
        }
        // every lane reads back exactly the logits it has just written
        if (p.sigmoid_bias)
            route_token_sigmoid(p.logits + static_cast<size_t>(t0 + t) * p.E, p.bias, p.multiplier, p.E, p.top_k, el,
                                p.ids_out + (t0 + t) * p.top_k, p.wts_out + (t0 + t) * p.top_k);
        else
            route_token(p.logits + static_cast<size_t>(t0 + t) * p.E, p.E, p.top_k, el, p.ids_out + (t0 + t) * p.top_k,
                        p.wts_out + (t0 + t) * p.top_k);
    }
    if (tid == 0) p.ticket[tg] = 0;  // ready for the next call
}

// Residual boundary of the reference's own layer form (muse_decode_layer/reference.py:339-344,452-455,473-476):
//   branch' = branch * (1 + branch_w)                      (optional)
//   s_out   = alpha * stream + beta * rmsnorm(branch', branch_eps),  (alpha, beta) from the gate; without a gate a plain add
//   normed  = bf16(rmsnorm(s_out, eps) * (1 + next_w)),   ssq[t] = sum s_out^2
// One block per token, the row in registers (H <= 8192).
struct BoundaryArgs {
    const float* stream;
    const void* branch;
    int branch_bf16, ldb;
    const __nv_bfloat16* branch_w;
    const __nv_bfloat16* gate;
    const __nv_bfloat16* next_w;
    float* s_out;
    __nv_bfloat16* normed;
    float* ssq;
    int H;
    float branch_eps, eps, temperature, gate_eps;
};

__device__ __forceinline__ float block_sum_256(float v, float* red) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    return ((red[0] + red[1]) + (red[2] + red[3])) + ((red[4] + red[5]) + (red[6] + red[7]));
}

__global__ void __launch_bounds__(256) boundary_kernel(BoundaryArgs p) {
    __shared__ float red[8];
    const int t = blockIdx.x, tid = threadIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    constexpr int kMaxVec = 8;
    float4 b[kMaxVec], s[kMaxVec];
    float bs = 0.0f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
        const int d = tid * 4 + i * 1024;
        b[i] = make_float4(0, 0, 0, 0), s[i] = make_float4(0, 0, 0, 0);
        if (d >= p.H) continue;
        s[i] = __ldcg(reinterpret_cast<const float4*>(p.stream + static_cast<size_t>(t) * p.H + d));
        if (p.branch_bf16) {
            const uint2 r = __ldcg(reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(p.branch) + static_cast<size_t>(t) * p.ldb + d));
            b[i] = make_float4(bf16lo(r.x), bf16hi(r.x), bf16lo(r.y), bf16hi(r.y));
        } else {
            b[i] = __ldcg(reinterpret_cast<const float4*>(static_cast<const float*>(p.branch) + static_cast<size_t>(t) * p.ldb + d));
        }
        if (p.branch_w != nullptr) {
            const uint2 w = *reinterpret_cast<const uint2*>(p.branch_w + d);
            b[i].x *= 1.0f + bf16lo(w.x), b[i].y *= 1.0f + bf16hi(w.x), b[i].z *= 1.0f + bf16lo(w.y), b[i].w *= 1.0f + bf16hi(w.y);
        }
        bs += b[i].x * b[i].x + b[i].y * b[i].y + b[i].z * b[i].z + b[i].w * b[i].w;
    }
    const float br = p.gate != nullptr ? rsqrtf(block_sum_256(bs, red) / p.H + p.branch_eps) : 1.0f;
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
        const int d = tid * 4 + i * 1024;
        if (d >= p.H) continue;
        float al[4] = {1.0f, 1.0f, 1.0f, 1.0f}, be[4] = {1.0f, 1.0f, 1.0f, 1.0f};
        if (p.gate != nullptr) {
            const uint2 g = *reinterpret_cast<const uint2*>(p.gate + d);
            const float gv[4] = {bf16lo(g.x), bf16hi(g.x), bf16lo(g.y), bf16hi(g.y)};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float w = gv[j] / p.temperature;
                be[j] = 1.0f / (1.0f + expf(-w));
                al[j] = sqrtf(fmaxf((1.0f / (1.0f + expf(w))) * (1.0f + be[j]), p.gate_eps));
            }
        }
        s[i].x = al[0] * s[i].x + be[0] * (b[i].x * br), s[i].y = al[1] * s[i].y + be[1] * (b[i].y * br);
        s[i].z = al[2] * s[i].z + be[2] * (b[i].z * br), s[i].w = al[3] * s[i].w + be[3] * (b[i].w * br);
        ss += s[i].x * s[i].x + s[i].y * s[i].y + s[i].z * s[i].z + s[i].w * s[i].w;
        if (p.s_out != nullptr) *reinterpret_cast<float4*>(p.s_out + static_cast<size_t>(t) * p.H + d) = s[i];
    }
    const float tot = block_sum_256(ss, red);
    if (tid == 0 && p.ssq != nullptr) p.ssq[t] = tot;
    if (p.normed == nullptr) return;
    const float rs = rsqrtf(tot / p.H + p.eps);
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
        const int d = tid * 4 + i * 1024;
        if (d >= p.H) continue;
        float f[4] = {1.0f, 1.0f, 1.0f, 1.0f};
        if (p.next_w != nullptr) {
            const uint2 w = *reinterpret_cast<const uint2*>(p.next_w + d);
            f[0] += bf16lo(w.x), f[1] += bf16hi(w.x), f[2] += bf16lo(w.y), f[3] += bf16hi(w.y);
        }
        *reinterpret_cast<uint2*>(p.normed + static_cast<size_t>(t) * p.H + d) =
            make_uint2(pack_bf16(s[i].x * rs * f[0], s[i].y * rs * f[1]), pack_bf16(s[i].z * rs * f[2], s[i].w * rs * f[3]));
    }
}

template <typename Kern, typename Args>
static int launch1(Kern kern, dim3 grid, dim3 block, int smem, cudaStream_t stream, int pdl, const Args& a) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, a) == cudaSuccess ? 0 : MSK_ERR_CUDA;
}

static int launch_prep(const float* stream, const void* w, void* xn, float* ssq, int T, int H, float eps, cudaStream_t s,
                       int pdl) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(T);
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, prep_norm_kernel, stream, static_cast<const __nv_bfloat16*>(w),
                              static_cast<__nv_bfloat16*>(xn), ssq, H, eps) == cudaSuccess
               ? 0
               : MSK_ERR_CUDA;
}

}  // namespace msk

extern "C" int msk_layer_front(const MskLayerFront* f, int* status, void* stream) {
    using namespace msk;
    if (f == nullptr || !f->stream || !f->input_norm_w || !f->w_qkv || !f->w_o || !f->pre_expert_norm_w || !f->router_w ||
        !f->xn0 || !f->ssq0 || !f->qkv || !f->attn || !f->stream1 || !f->xn1 || !f->ssq1 || !f->router_part ||
        !f->router_ticket || !f->logits || !f->topk_ids || !f->topk_weights)
        return MSK_ERR_INVALID;
    const int T = f->B * f->L, H = f->H, nqkv = (2 * f->Hq + 2 * f->Hkv) * f->d, no = f->Hq * f->d;
    if (T < 1 || T > 256 || H % 1024 != 0 || H > 8192 || f->E < 1 || f->E > 256 || f->top_k < 1 ||
        f->top_k > 8 || f->top_k > f->E)
        return MSK_ERR_UNSUPPORTED;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int rc = launch_prep(f->stream, f->input_norm_w, f->xn0, f->ssq0, T, H, f->norm_eps, s, f->pdl);
    if (rc != 0) return rc;

    MskProjParams q = {};
    q.x = f->xn0, q.w = f->w_qkv, q.M = T, q.N = nqkv, q.K = H, q.splits = f->qkv_splits;
    q.out = f->qkv, q.out_fp32 = 0, q.ldo = nqkv;
    q.scratch = f->qkv_scratch, q.scratch_bytes = f->qkv_scratch_bytes;
    q.pdl = 1;
    rc = msk_proj_skinny(&q, status, stream);
    if (rc != 0) return rc;

    MskAttnParams a = {};
    a.qkv = f->qkv, a.ld_qkv = nqkv, a.out = f->attn, a.ld_out = no;
    a.k_cache = f->k_cache, a.v_cache = f->v_cache, a.k_scale = f->k_scale, a.v_scale = f->v_scale;
    a.seq_lens = f->seq_lens, a.page_table = f->page_table, a.max_pages = f->max_pages, a.cache_loc = f->cache_loc;
    a.inv_freq = f->inv_freq, a.B = f->B, a.L = f->L, a.Hq = f->Hq, a.Hkv = f->Hkv, a.d = f->d;
    a.page_size = f->page_size, a.num_pages = f->num_pages, a.window = f->window;
    a.qk_scale_factor = f->qk_scale_factor, a.sm_scale = f->sm_scale;
    a.chunks = f->attn_chunks, a.stages = f->attn_stages, a.issuers = f->attn_issuers, a.row_groups = f->attn_row_groups, a.pdl = 1;
    rc = msk_attn_decode(&a, status, stream);
    if (rc != 0) return rc;

    MskProjParams o = {};
    o.x = f->attn, o.w = f->w_o, o.M = T, o.N = H, o.K = no, o.splits = f->o_splits;
    o.out = f->stream1, o.out_fp32 = 1, o.ldo = H;
    o.resid = f->stream, o.ldr = H;
    o.scratch = f->o_scratch, o.scratch_bytes = f->o_scratch_bytes;
    o.next_norm_w = f->pre_expert_norm_w, o.out_normed = f->xn1, o.ldn = H, o.normed_fp16 = 1, o.out_ssq = f->ssq1, o.pdl = 1;
    rc = msk_proj_skinny(&o, status, stream);
    if (rc != 0) return rc;

    MskRouterParams r = {};
    r.x = f->stream1, r.norm_w = f->pre_expert_norm_w, r.ssq = f->ssq1, r.ssq_parts = (H + 127) / 128, r.eps = f->norm_eps;
    r.router_w = f->router_w, r.router_bias = f->router_bias, r.E = f->E, r.T = T, r.H = H, r.top_k = f->top_k;
    r.part = f->router_part, r.ticket = f->router_ticket, r.logits = f->logits;
    r.topk_ids = f->topk_ids, r.topk_weights = f->topk_weights, r.pdl = 1;
    return msk_router(&r, status, stream);
}

extern "C" int msk_router(const MskRouterParams* q, int* status, void* stream) {
    using namespace msk;
    (void)status;
    if (q == nullptr || !q->x || !q->norm_w || !q->ssq || !q->router_w || !q->part || !q->ticket || !q->logits || !q->topk_ids ||
        !q->topk_weights)
        return MSK_ERR_INVALID;
    if (q->T < 1 || q->H % 1024 != 0 || q->H > 8192 || q->E < 1 || q->E > 256 || q->top_k < 1 || q->top_k > 8 || q->top_k > q->E ||
        q->ssq_parts < 1)
        return MSK_ERR_UNSUPPORTED;
    RouterArgs r = {};
    r.s1 = q->x, r.w = static_cast<const __nv_bfloat16*>(q->norm_w), r.ssq = q->ssq;
    r.ssq_parts = q->ssq_parts, r.eps = q->eps, r.R = q->router_w, r.bias = q->router_bias;
    r.part = q->part, r.ticket = q->ticket, r.logits = q->logits, r.T = q->T, r.H = q->H, r.E = q->E;
    r.top_k = q->top_k, r.ids_out = q->topk_ids, r.wts_out = q->topk_weights;
    r.sigmoid_bias = q->sigmoid_bias, r.multiplier = q->multiplier;
    const int et = (q->E + kRouterE - 1) / kRouterE, n_tg = (q->T + kRouterT - 1) / kRouterT;
    if (n_tg >= 3 && q->E <= kWideE) {
        // many tokens (measured: from three token groups on): whole expert range per block, about one block per SM
        int tiles = q->H / kRouterK, ph = 1;
        while (n_tg * (tiles / ph) > 160 && (tiles / ph) % 2 == 0) ph *= 2;
        r.phases = ph;
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MSK_ERR_CUDA;
        static bool configured[64] = {};  // per device, like the attribute itself
        if (!configured[dev]) {
            if (cudaFuncSetAttribute(router_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kRouterWideSmem) != cudaSuccess)
                return MSK_ERR_CUDA;
            configured[dev] = true;
        }
        return launch1(router_wide_kernel, dim3(tiles / ph, n_tg), dim3(256), kRouterWideSmem, static_cast<cudaStream_t>(stream), q->pdl, r);
    }
    // few tokens: as many K splits as there are 128-k tiles (the 2 MB of router weights spread over the SMs);
    // four token groups or more: blocks of four tiles (the K-split count must stay a multiple of 8)
    r.phases = (n_tg >= 4 && (q->H / kRouterK) % 32 == 0) ? 4 : 1;
    const int ks = q->H / (kRouterK * r.phases);  // <= 64
    // one block per token group: letting a block walk several groups so that the grid stays within one wave of
    // CTAs measured slower (each group is a chain of global round trips; 55 against 45 us at 256 tokens)
    return launch1(router_kernel, dim3(ks, et, n_tg), dim3(256), 0, static_cast<cudaStream_t>(stream), q->pdl, r);
}

extern "C" int msk_residual_boundary(const MskBoundaryParams* q, void* stream) {
    using namespace msk;
    if (q == nullptr || !q->stream || !q->branch || q->T < 1 || q->H < 4 || q->H % 4 != 0 || q->H > 8192 || q->ldb % 4 != 0)
        return MSK_ERR_INVALID;
    BoundaryArgs a = {};
    a.stream = q->stream, a.branch = q->branch, a.branch_bf16 = q->branch_bf16, a.ldb = q->ldb > 0 ? q->ldb : q->H;
    a.branch_w = static_cast<const __nv_bfloat16*>(q->branch_w), a.gate = static_cast<const __nv_bfloat16*>(q->gate);
    a.next_w = static_cast<const __nv_bfloat16*>(q->next_norm_w), a.s_out = q->stream_out;
    a.normed = static_cast<__nv_bfloat16*>(q->normed_out), a.ssq = q->ssq_out, a.H = q->H;
    a.branch_eps = q->branch_eps, a.eps = q->eps, a.temperature = q->temperature > 0.0f ? q->temperature : 0.3f;
    a.gate_eps = q->gate_eps;
    return launch1(boundary_kernel, dim3(q->T), dim3(256), 0, static_cast<cudaStream_t>(stream), q->pdl, a);
}

extern "C" int msk_rmsnorm(const float* x, const void* w, void* out_bf16, float* ssq, int T, int H, float eps, int pdl, void* stream) {
    using namespace msk;
    if (!x || !w || !out_bf16 || !ssq || T < 1 || H < 4 || H % 4 != 0 || H > 8192) return MSK_ERR_INVALID;
    return launch_prep(x, w, out_bf16, ssq, T, H, eps, static_cast<cudaStream_t>(stream), pdl);
}

extern "C" int msk_layer_decode(const MskLayerParams* p, int* status, void* stream) {
    if (p == nullptr) return MSK_ERR_INVALID;
    int rc = msk_layer_front(&p->front, status, stream);
    if (rc != 0) return rc;
    MskMoeParams m = p->moe;
    const MskLayerFront& f = p->front;
    m.x = f.xn1, m.ldx = f.H, m.x_fp16 = 1;
    m.x_ssq = f.ssq1 + static_cast<size_t>((f.H + 127) / 128) * (f.B * f.L), m.x_ssq_parts = 1,  // the router's totals
     m.x_inv_dim = 1.0f / f.H, m.x_eps = f.norm_eps;
    m.logits = nullptr, m.topk_ids = f.topk_ids, m.topk_weights = f.topk_weights, m.top_k = f.top_k, m.ld_topk = 0;
    m.T = f.B * f.L, m.H = f.H;
    m.resid = f.stream1, m.ldr = f.H;
    m.pdl = 1;
    return msk_moe_forward(&m, status, stream);
}

// Skinny BF16 projection out[M, N] = x[M, K] * W[N, K]^T for M <= 256 tokens (decode / verify).
//
// Swap-AB: the 128 weight rows of a CTA's tile are the UMMA M side, the tokens the N side, so the
// tensor-core tile is full however few tokens there are.  One CTA = (128-row tile, K split, token split),
// 256 threads.  Few tokens: the K range of a tile is split over CTAs until tiles x splits fills the SMs (FP32
// partial tiles meet in L2).  Many tokens (verify blocks, 256 requests): the tokens are split instead, so that
// every CTA streams less of x per weight byte and finishes its own tokens straight from tensor memory.
//   warp 0 / one lane   TMA producer: W tile [128 x 64] and x tile [bn x 64] per stage, 128-byte swizzle,
//                       ring of up to 12 stages (>= 200 KB in flight per SM).  The W stream starts before
//                       anything else in the CTA and before the programmatic-dependent-launch wait; only x
//                       depends on the previous kernel.
//   warp 1 / one lane   tcgen05.mma kind::f16 (BF16 x BF16 -> FP32 in TMEM), 4 per stage; tcgen05.commit
//                       hands each ring slot back to the producer.
//   all 8 warps         epilogue: tcgen05.ld (lane = weight row; warps w and w + 4 share a lane quarter and
//                       split the tokens).  With K splits every CTA stores its FP32 partial tile to a scratch
//                       buffer (L2) and takes a ticket per tile; the CTA that draws the last ticket adds all
//                       partials in split order (bitwise reproducible whoever is last), applies the fused
//                       epilogue and stores.  The split count is free (not tied to a cluster shape): it is
//                       chosen so that tiles x splits fills the SMs.
// The epilogue works on blocks of 8 tokens with every load of a block issued before the first use: with two
// warps per scheduler each instruction's latency is exposed, so dependent one-token-at-a-time code is what
// costs (measured: 400 clocks per token that way).
// HBM traffic: W once (N*K*2 bytes); x is re-read per tile from L2.  Roofline: HBM.
#include <cuda_fp16.h>

#include "msk.h"
#include "ptx.cuh"
#include "tmap.cuh"

namespace msk {

constexpr int kProjMaxStages = 12;
constexpr int kProjWBytes = 128 * 128;  // one W stage: 128 rows x 64 bf16
constexpr int kProjThreads = 256;
constexpr int kProjMaxSplits = 16;
constexpr int kProjTicketBytes = 4096;  // 1024 tile tickets at the start of the scratch buffer
constexpr int kProjMaxDevices = 64;

struct ProjArgs {
    int M, N, K, bn, nstages;  // bn: tokens per CTA (multiple of 16)
    int Mtot;                  // all tokens of the launch (M is this CTA's share once the kernel has offset its views)
    uint32_t tmem_cols;
    void* out;
    int out_fp32, ldo;
    const float* in_ssq;
    int in_ssq_parts;
    float in_inv_dim, in_eps;
    const float* resid;
    int ldr;
    const __nv_bfloat16* next_norm_w;
    __nv_bfloat16* out_normed;
    int ldn, normed_fp16;
    float* out_ssq;
    float* part;    // [tiles][token splits][S][bn / 4][128 rows][4 tokens] FP32 partial tiles (S > 1): a warp's float4 accesses
                    // (lane = row) are 512 contiguous bytes
    int* ticket;    // [tiles][token splits], zero between launches
    int* status;
};

// Sum over the 32 lanes of 8 values per lane in 9 shuffles (instead of 40): the first three steps halve the
// number of values a lane carries, the last two are plain butterflies.  Afterwards every lane holds the total
// of value index ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1).
__device__ __forceinline__ float warp_sum8(const float (&v)[8], int lane) {
    float a[4], b[2], c;
    const bool h16 = lane & 16, h8 = lane & 8, h4 = lane & 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float keep = h16 ? v[4 + i] : v[i], give = h16 ? v[i] : v[4 + i];
        a[i] = keep + __shfl_xor_sync(0xffffffffu, give, 16);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float keep = h8 ? a[2 + i] : a[i], give = h8 ? a[i] : a[2 + i];
        b[i] = keep + __shfl_xor_sync(0xffffffffu, give, 8);
    }
    {
        const float keep = h4 ? b[1] : b[0], give = h4 ? b[0] : b[1];
        c = keep + __shfl_xor_sync(0xffffffffu, give, 4);
    }
    c += __shfl_xor_sync(0xffffffffu, c, 2);
    c += __shfl_xor_sync(0xffffffffu, c, 1);
    return c;
}

struct EpiCtx {
    bool in_n, ok;
    int n, lane, S, bn;
    uint32_t trow;
    float nw;
    const float* parts;  // this row's partial sums of split 0, tokens 0..3 (token group g: + g * 512, split r: + r * 128 * bn)
    const float* rs;     // [256] input row scales (shared memory)
    float* wsum;         // [256] this lane quarter's sums of squares (shared memory)
};

// Fused epilogue for NB blocks of 8 tokens starting at t0, thread = weight row.  Every global load of the
// blocks (residual, partial sums of two splits at a time) is issued before the first is used: one exposed L2
// round trip per 8 * NB tokens instead of one per token.
template <int NB>
__device__ __forceinline__ void finish_block(const ProjArgs& p, const EpiCtx& c, int t0) {
    constexpr int NT = 8 * NB;
    float rv[NT], acc[NT];
#pragma unroll
    for (int i = 0; i < NT; ++i)
        rv[i] = (p.resid != nullptr && c.in_n && t0 + i < p.M) ? __ldcg(p.resid + static_cast<size_t>(t0 + i) * p.ldr + c.n) : 0.0f;
    if (c.S > 1) {
#pragma unroll
        for (int i = 0; i < NT; ++i) acc[i] = 0.0f;
#pragma unroll 1
        constexpr int NS = NB == 1 ? 4 : 2;  // splits whose loads are in flight together; added in split order
        for (int r0 = 0; r0 < c.S; r0 += NS) {
            float4 a[NS][2 * NB];
#pragma unroll
            for (int j = 0; j < NS; ++j) {
                const float* src = c.parts + static_cast<size_t>(min(r0 + j, c.S - 1)) * 128 * c.bn + (t0 >> 2) * 512;
#pragma unroll
                for (int q = 0; q < 2 * NB; ++q) a[j][q] = __ldcg(reinterpret_cast<const float4*>(src + q * 512));
            }
#pragma unroll
            for (int j = 0; j < NS; ++j) {
                if (r0 + j >= c.S) break;
#pragma unroll
                for (int q = 0; q < 2 * NB; ++q)
                    acc[4 * q] += a[j][q].x, acc[4 * q + 1] += a[j][q].y, acc[4 * q + 2] += a[j][q].z, acc[4 * q + 3] += a[j][q].w;
            }
        }
    } else {
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            uint32_t v[8];
            tmem_ld8(c.trow + t0 + 8 * b, v);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[8 * b + i] = __uint_as_float(v[i]);
        }
        tmem_wait_ld();
    }
#pragma unroll
    for (int q = 0; q < 2 * NB; ++q) {
        const float4 r = *reinterpret_cast<const float4*>(c.rs + t0 + 4 * q);
        acc[4 * q] = c.in_n ? acc[4 * q] * r.x + rv[4 * q] : 0.0f;
        acc[4 * q + 1] = c.in_n ? acc[4 * q + 1] * r.y + rv[4 * q + 1] : 0.0f;
        acc[4 * q + 2] = c.in_n ? acc[4 * q + 2] * r.z + rv[4 * q + 2] : 0.0f;
        acc[4 * q + 3] = c.in_n ? acc[4 * q + 3] * r.w + rv[4 * q + 3] : 0.0f;
    }
    if (c.in_n && c.ok) {
        if (p.out != nullptr) {
            if (p.out_fp32) {
#pragma unroll
                for (int i = 0; i < NT; ++i)
                    if (t0 + i < p.M) static_cast<float*>(p.out)[static_cast<size_t>(t0 + i) * p.ldo + c.n] = acc[i];
            } else {
#pragma unroll
                for (int i = 0; i < NT; ++i)
                    if (t0 + i < p.M) static_cast<__nv_bfloat16*>(p.out)[static_cast<size_t>(t0 + i) * p.ldo + c.n] = __float2bfloat16(acc[i]);
            }
        }
        if (p.out_normed != nullptr) {
            if (p.normed_fp16) {
#pragma unroll
                for (int i = 0; i < NT; ++i)
                    if (t0 + i < p.M)
                        reinterpret_cast<__half*>(p.out_normed)[static_cast<size_t>(t0 + i) * p.ldn + c.n] =
                            __float2half_rn(fminf(fmaxf(acc[i] * c.nw, -65504.0f), 65504.0f));
            } else {
#pragma unroll
                for (int i = 0; i < NT; ++i)
                    if (t0 + i < p.M) p.out_normed[static_cast<size_t>(t0 + i) * p.ldn + c.n] = __float2bfloat16(acc[i] * c.nw);
            }
        }
    }
    if (p.out_ssq != nullptr) {
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            float sq[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) sq[i] = acc[8 * b + i] * acc[8 * b + i];
            const float tot = warp_sum8(sq, c.lane);
            if ((c.lane & 3) == 0) c.wsum[t0 + 8 * b + ((c.lane >> 4) & 1) * 4 + ((c.lane >> 3) & 1) * 2 + ((c.lane >> 2) & 1)] = tot;
        }
    }
}

__global__ void __launch_bounds__(kProjThreads) proj_skinny_kernel(const __grid_constant__ CUtensorMap tm_w,
                                                                   const __grid_constant__ CUtensorMap tm_x, const ProjArgs pa) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * kProjMaxStages + 1];
    __shared__ uint32_t tmem_slot;
    __shared__ int last_s;
    __shared__ __align__(16) float rs[256];
    __shared__ float wsum[4][256];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = gridDim.x, rank = blockIdx.x, tile = blockIdx.y;
    const int n0 = tile * 128;
    // this CTA's token share: every per-token pointer is moved to its first token
    const int tok0 = blockIdx.z * pa.bn;
    ProjArgs p = pa;
    p.M = max(0, min(pa.bn, pa.M - tok0));
    if (p.out != nullptr) p.out = static_cast<char*>(p.out) + static_cast<size_t>(tok0) * p.ldo * (p.out_fp32 ? 4 : 2);
    if (p.resid != nullptr) p.resid += static_cast<size_t>(tok0) * p.ldr;
    if (p.out_normed != nullptr) p.out_normed += static_cast<size_t>(tok0) * p.ldn;
    if (p.in_ssq != nullptr) p.in_ssq += tok0;
    if (p.out_ssq != nullptr) p.out_ssq += tok0;
    const int unit = tile * gridDim.z + blockIdx.z;  // (tile, token split): owns a ticket and S partial tiles
    const int where = (MSK_K_PROJ << 8);
    const int nst = p.nstages, bn = p.bn;
    const uint32_t stage_bytes = kProjWBytes + bn * 128;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int KT = p.K / 64;
    const int kt0 = static_cast<int>(static_cast<long long>(rank) * KT / S);
    const int kt1 = static_cast<int>(static_cast<long long>(rank + 1) * KT / S);
    const int nk = kt1 - kt0;
    // Every tile of a K split reads the same x tiles; started together they would all pull the same lines out of
    // the same L2 slices at the same time.  Tile y therefore walks its K range from a different starting point.
    const int rot = nk > 0 ? static_cast<int>((blockIdx.y * 5u) % static_cast<unsigned>(nk)) : 0;
    auto kt_of = [&](int i) { const int j = i + rot; return kt0 + (j >= nk ? j - nk : j); };
    auto full = [&](int s) { return smem_u32(&bars[s]); };
    auto empty = [&](int s) { return smem_u32(&bars[kProjMaxStages + s]); };
    const uint32_t bar_done = smem_u32(&bars[2 * kProjMaxStages]);
    const int pre = nk < nst ? nk : nst;

    // The producer thread sets up the barriers itself and starts the weight stream before the CTA's first
    // barrier: the first bytes' DRAM latency is the longest single item of a small launch.
    if (tid == 0) {
        prefetch_tmap(&tm_w);
        prefetch_tmap(&tm_x);
        for (int s = 0; s < nst; ++s) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), 1);
        }
        mbar_init(bar_done, 1);
        fence_mbar_init();
        for (int i = 0; i < pre; ++i) {
            mbar_expect_tx(full(i), stage_bytes);
            tma_load_2d(base + i * stage_bytes, &tm_w, full(i), kt_of(i) * 64, n0);
        }
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_slot), p.tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    pdl_launch_dependents();

    if (warp == 0) {
        if (lane == 0) {
            pdl_wait();  // x is the previous kernel's output
            for (int i = 0; i < pre; ++i)
                tma_load_2d(base + i * stage_bytes + kProjWBytes, &tm_x, full(i), kt_of(i) * 64, tok0);
            int s = 0, ph = 0;  // ring slot of k-step i and the parity of its previous use
            for (int i = pre; i < nk; ++i) {
                if (!mbar_wait(empty(s), ph, p.status, where | 1)) break;
                mbar_expect_tx(full(s), stage_bytes);
                tma_load_2d(base + s * stage_bytes, &tm_w, full(s), kt_of(i) * 64, n0);
                tma_load_2d(base + s * stage_bytes + kProjWBytes, &tm_x, full(s), kt_of(i) * 64, tok0);
                if (++s == nst) s = 0, ph ^= 1;
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(128, bn, 1, 1, 0, 0);
            bool mok = true;
            int s = 0, ph = 0;
            for (int i = 0; i < nk && mok; ++i) {
                mok = mbar_wait(full(s), ph, p.status, where | 2);
                if (!mok) break;
                tc_fence_after();
                const uint32_t a = base + s * stage_bytes;
                const uint64_t ad = umma_smem_desc(a, 16, 1024, kSwizzle128);
                const uint64_t bd = umma_smem_desc(a + kProjWBytes, 16, 1024, kSwizzle128);
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_f16_ss(tmem, ad + 2 * k, bd + 2 * k, idesc, (i | k) != 0);
                umma_commit(empty(s));
                if (++s == nst) s = 0, ph ^= 1;
            }
            if (mok) umma_commit(bar_done);
        }
        __syncwarp();
    }

    // ---------------- epilogue: lane = weight row, warps w and w + 4 split the tokens
    pdl_wait();
    for (int t = tid; t < 256; t += kProjThreads) {
        float r = 1.0f;
        if (p.in_ssq != nullptr && t < p.M) {
            float s = 0.0f;
            for (int part = 0; part < p.in_ssq_parts; ++part) s += __ldcg(p.in_ssq + part * p.Mtot + t);
            r = rsqrtf(s * p.in_inv_dim + p.in_eps);
        }
        rs[t] = r;
    }
    const bool ok = nk > 0 && mbar_wait(bar_done, 0, p.status, where | 3);
    tc_fence_after();
    __syncthreads();
    const int quarter = warp & 3, row = quarter * 32 + lane, n = n0 + row;
    const uint32_t trow = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
    const int half = bn >> 1;                                  // bn is a multiple of 16
    const int t_begin = (warp >> 2) * half, t_end = t_begin + half;

    bool fin = true;  // this CTA finishes the tile
    if (S > 1) {
        float* mine = p.part + (static_cast<size_t>(unit) * S + rank) * 128 * bn + row * 4;  // token group g: + g * 512
        int t0 = t_begin;
#pragma unroll 1
        for (; t0 + 32 <= t_end; t0 += 32) {  // one tensor-memory round trip per 32 tokens
            uint32_t v[4][8];
#pragma unroll
            for (int b = 0; b < 4; ++b) tmem_ld8(trow + t0 + 8 * b, v[b]);
            tmem_wait_ld();
            float* dst = mine + (t0 >> 2) * 512;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                *reinterpret_cast<float4*>(dst + (2 * b) * 512) = make_float4(__uint_as_float(v[b][0]), __uint_as_float(v[b][1]), __uint_as_float(v[b][2]), __uint_as_float(v[b][3]));
                *reinterpret_cast<float4*>(dst + (2 * b + 1) * 512) = make_float4(__uint_as_float(v[b][4]), __uint_as_float(v[b][5]), __uint_as_float(v[b][6]), __uint_as_float(v[b][7]));
            }
        }
#pragma unroll 1
        for (; t0 < t_end; t0 += 8) {
            uint32_t v[8];
            tmem_ld8(trow + t0, v);
            tmem_wait_ld();
            float* dst = mine + (t0 >> 2) * 512;
            *reinterpret_cast<float4*>(dst) = make_float4(__uint_as_float(v[0]), __uint_as_float(v[1]), __uint_as_float(v[2]), __uint_as_float(v[3]));
            *reinterpret_cast<float4*>(dst + 512) = make_float4(__uint_as_float(v[4]), __uint_as_float(v[5]), __uint_as_float(v[6]), __uint_as_float(v[7]));
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const int old = atomicAdd(p.ticket + unit, 1);
            last_s = old == S - 1;
            if (old == S - 1) p.ticket[unit] = 0;  // ready for the next launch
        }
        __syncthreads();
        fin = last_s != 0;
        if (fin) __threadfence();
    }

    if (fin) {
        EpiCtx c;
        c.in_n = n < p.N, c.ok = ok, c.n = n, c.lane = lane, c.S = S, c.bn = bn, c.trow = trow;
        c.nw = (p.next_norm_w != nullptr && c.in_n) ? 1.0f + __bfloat162float(p.next_norm_w[n]) : 1.0f;
        c.parts = p.part + static_cast<size_t>(unit) * S * 128 * bn + row * 4;
        c.rs = rs, c.wsum = wsum[quarter];
        const int t_stop = min(t_end, (p.M + 7) & ~7);
        int t0 = t_begin;
#pragma unroll 1
        for (; t0 + 32 <= t_stop; t0 += 32) finish_block<4>(p, c, t0);
#pragma unroll 1
        for (; t0 < t_stop; t0 += 8) finish_block<1>(p, c, t0);
        if (p.out_ssq != nullptr) {
            __syncthreads();
            if (ok)
                for (int t = tid; t < p.M; t += kProjThreads)
                    p.out_ssq[tile * p.Mtot + t] = (wsum[0][t] + wsum[1][t]) + (wsum[2][t] + wsum[3][t]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, p.tmem_cols);
}

// Ways to split a launch so that tiles x token splits x K splits fills the SMs.  Token splits first when there
// are many tokens (at least 64 per CTA): they need no reduction and cut the x bytes a CTA streams per weight
// byte; K splits (at least 4 k-steps each) take the rest.
struct ProjPlan {
    int S, St, bn;  // K splits, token splits, tokens per CTA (multiple of 16)
};
static ProjPlan plan_launch(int M, int tiles, int KT, int sms, int splits, int token_splits) {
    int ways = sms / tiles;
    if (ways < 1) ways = 1;
    int St = token_splits > 0 ? token_splits : min(ways, max(1, M / 64));
    if (St > (M + 15) / 16) St = (M + 15) / 16;
    int bn = ((M + St - 1) / St + 15) / 16 * 16;
    St = (M + bn - 1) / bn;  // no empty share
    int S = splits;
    if (S <= 0) {
        S = ways / St;
        if (S > KT / 4) S = KT / 4;
        if (S > kProjMaxSplits) S = kProjMaxSplits;
        if (S < 1) S = 1;
    }
    if (S > KT) S = KT;
    return {S, St, bn};
}

}  // namespace msk

static size_t plan_scratch_bytes(const msk::ProjPlan& pl, int tiles) {
    return msk::kProjTicketBytes + (pl.S > 1 ? static_cast<size_t>(tiles) * pl.St * pl.S * 128 * pl.bn * sizeof(float) : 0);
}

extern "C" int msk_proj_scratch_bytes(int M, int N, int K, int splits, int token_splits, size_t* bytes) {
    using namespace msk;
    if (M < 1 || M > 256 || N < 1 || K < 64 || K % 64 != 0 || bytes == nullptr) return MSK_ERR_INVALID;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int tiles = (N + 127) / 128, KT = K / 64;
    const ProjPlan pl = plan_launch(M, tiles, KT, sms, splits, token_splits);
    if (tiles * pl.St > kProjTicketBytes / 4) return MSK_ERR_UNSUPPORTED;
    *bytes = plan_scratch_bytes(pl, tiles);
    return 0;
}

extern "C" int msk_proj_skinny(const MskProjParams* q, int* status, void* stream) {
    using namespace msk;
    if (q == nullptr || q->x == nullptr || q->w == nullptr) return MSK_ERR_INVALID;
    if (q->M < 1 || q->M > 256 || q->N < 1 || q->K < 64 || q->K % 64 != 0) return MSK_ERR_UNSUPPORTED;
    if (q->out == nullptr && q->out_normed == nullptr) return MSK_ERR_INVALID;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kProjMaxDevices) return MSK_ERR_CUDA;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int tiles = (q->N + 127) / 128, KT = q->K / 64;
    if (q->splits > kProjMaxSplits || q->token_splits > 16) return MSK_ERR_UNSUPPORTED;
    const ProjPlan pl = plan_launch(q->M, tiles, KT, sms, q->splits, q->token_splits);
    if (tiles * pl.St > kProjTicketBytes / 4) return MSK_ERR_UNSUPPORTED;
    const int S = pl.S, bn = pl.bn;
    if (S > 1) {
        if (q->scratch == nullptr || q->scratch_bytes < plan_scratch_bytes(pl, tiles)) return MSK_ERR_INVALID;
        if ((reinterpret_cast<uintptr_t>(q->scratch) & 15) != 0) return MSK_ERR_INVALID;
    }
    uint32_t cols = 32;
    while (cols < static_cast<uint32_t>(bn)) cols *= 2;
    const int stage = kProjWBytes + bn * 128;
    const int budget = 232448 - 8192 - 1024;  // opt-in limit minus static shared memory and alignment slack
    int nst = budget / stage;
    if (nst > kProjMaxStages) nst = kProjMaxStages;
    const int per_cta = (KT + S - 1) / S;
    if (nst > per_cta) nst = per_cta;
    if (nst < 2 && per_cta >= 2) return MSK_ERR_UNSUPPORTED;
    const int smem = 1024 + nst * stage;

    CUtensorMap tm_w, tm_x;
    int rc = make_tmap_bf16_2d(&tm_w, q->w, q->N, q->K, q->K, 128);
    if (rc == 0) rc = make_tmap_bf16_2d(&tm_x, q->x, q->M, q->K, q->K, bn);
    if (rc != 0) return rc;

    ProjArgs a{};
    a.M = q->M, a.Mtot = q->M, a.N = q->N, a.K = q->K, a.bn = bn, a.nstages = nst, a.tmem_cols = cols;
    a.out = q->out, a.out_fp32 = q->out_fp32, a.ldo = q->ldo;
    a.in_ssq = q->in_ssq, a.in_ssq_parts = q->in_ssq_parts, a.in_inv_dim = q->in_inv_dim, a.in_eps = q->in_eps;
    a.resid = q->resid, a.ldr = q->ldr;
    a.next_norm_w = static_cast<const __nv_bfloat16*>(q->next_norm_w);
    a.out_normed = static_cast<__nv_bfloat16*>(q->out_normed), a.ldn = q->ldn, a.normed_fp16 = q->normed_fp16;
    a.out_ssq = q->out_ssq, a.status = status;
    a.ticket = static_cast<int*>(q->scratch);
    a.part = q->scratch != nullptr ? reinterpret_cast<float*>(static_cast<char*>(q->scratch) + kProjTicketBytes) : nullptr;

    static int configured_smem[kProjMaxDevices] = {};  // the attribute is per device
    if (smem > configured_smem[dev]) {
        if (cudaFuncSetAttribute(proj_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return MSK_ERR_CUDA;
        configured_smem[dev] = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(S, tiles, pl.St);
    cfg.blockDim = dim3(kProjThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attrs[1];
    attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = q->pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, proj_skinny_kernel, tm_w, tm_x, a);
    return e == cudaSuccess ? 0 : MSK_ERR_CUDA;
}

// Skinny BF16 projection out[M, N] = x[M, K] * W[N, K]^T for M <= 256 tokens (decode / verify).
//
// Swap-AB: the 128 weight rows of a CTA's tile are the UMMA M side, the tokens the N side, so the
// tensor-core tile is full however few tokens there are.  One CTA = (128-row tile, K split).
//   warp 0 / one lane   TMA producer: W tile [128 x 64] and x tile [bn x 64] per stage, 128-byte swizzle,
//                       ring of up to 12 stages (>= 200 KB in flight per SM).  The W stream starts before
//                       the programmatic-dependent-launch wait; only x depends on the previous kernel.
//   warp 1 / one lane   tcgen05.mma kind::f16 (BF16 x BF16 -> FP32 in TMEM), 4 per stage; tcgen05.commit
//                       hands each ring slot back to the producer.
//   all 4 warps         epilogue: tcgen05.ld (lane = weight row).  The K splits of one tile form a thread
//                       block cluster; every CTA pushes its partial sums for the tokens another CTA owns
//                       straight into that CTA's shared memory (DSMEM), one cluster barrier, then each owner
//                       adds in a fixed order (bitwise reproducible), applies the fused epilogue and stores.
// HBM traffic: W once (N*K*2 bytes); x is re-read per tile from L2.  Roofline: HBM.
#include <cuda_fp16.h>

#include "msk.h"
#include "ptx.cuh"
#include "tmap.cuh"

namespace msk {

constexpr int kProjMaxStages = 12;
constexpr int kProjWBytes = 128 * 128;  // one W stage: 128 rows x 64 bf16

struct ProjArgs {
    int M, N, K, bn, nstages, red_rows;
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
    int* status;
};

__global__ void __launch_bounds__(128) proj_skinny_kernel(const __grid_constant__ CUtensorMap tm_w,
                                                          const __grid_constant__ CUtensorMap tm_x, ProjArgs p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * kProjMaxStages + 1];
    __shared__ uint32_t tmem_slot;
    __shared__ float rs[256];
    __shared__ float wsum[4][256];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = gridDim.x, rank = blockIdx.x;  // the cluster spans the whole x extent of the grid
    const int n0 = blockIdx.y * 128;
    const int where = (MSK_K_PROJ << 8);
    const int nst = p.nstages, bn = p.bn;
    const uint32_t stage_bytes = kProjWBytes + bn * 128;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t red_base = base + nst * stage_bytes;
    const float* red = reinterpret_cast<const float*>(smem_raw + (red_base - smem_u32(smem_raw)));
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

    if (warp == 0) {
        tmem_alloc(smem_u32(&tmem_slot), p.tmem_cols);
        tmem_relinquish();
    }
    if (tid == 32) {
        for (int s = 0; s < nst; ++s) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), 1);
        }
        mbar_init(bar_done, 1);
        fence_mbar_init();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    pdl_launch_dependents();

    if (warp == 0) {
        if (lane == 0) {
            prefetch_tmap(&tm_w);
            prefetch_tmap(&tm_x);
            const int pre = nk < nst ? nk : nst;
            for (int i = 0; i < pre; ++i) {
                mbar_expect_tx(full(i), stage_bytes);
                tma_load_2d(base + i * stage_bytes, &tm_w, full(i), kt_of(i) * 64, n0);
            }
            pdl_wait();  // x is the previous kernel's output
            for (int i = 0; i < pre; ++i)
                tma_load_2d(base + i * stage_bytes + kProjWBytes, &tm_x, full(i), kt_of(i) * 64, 0);
            for (int i = pre; i < nk; ++i) {
                const int s = i % nst;
                if (!mbar_wait(empty(s), ((i / nst) - 1) & 1, p.status, where | 1)) break;
                mbar_expect_tx(full(s), stage_bytes);
                tma_load_2d(base + s * stage_bytes, &tm_w, full(s), kt_of(i) * 64, n0);
                tma_load_2d(base + s * stage_bytes + kProjWBytes, &tm_x, full(s), kt_of(i) * 64, 0);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(128, bn, 1, 1, 0, 0);
            bool ok = true;
            for (int i = 0; i < nk && ok; ++i) {
                const int s = i % nst;
                ok = mbar_wait(full(s), (i / nst) & 1, p.status, where | 2);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a = base + s * stage_bytes;
                const uint64_t ad = umma_smem_desc(a, 16, 1024, kSwizzle128);
                const uint64_t bd = umma_smem_desc(a + kProjWBytes, 16, 1024, kSwizzle128);
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_f16_ss(tmem, ad + 2 * k, bd + 2 * k, idesc, (i | k) != 0);
                umma_commit(empty(s));
            }
            if (ok) umma_commit(bar_done);
        }
        __syncwarp();
    }

    // ---------------- epilogue: all four warps, lane = weight row
    pdl_wait();
    for (int t = tid; t < bn; t += 128) {
        float r = 1.0f;
        if (p.in_ssq != nullptr && t < p.M) {
            float s = 0.0f;
            for (int part = 0; part < p.in_ssq_parts; ++part) s += __ldcg(p.in_ssq + part * p.M + t);
            r = rsqrtf(s * p.in_inv_dim + p.in_eps);
        }
        rs[t] = r;
    }
    const bool ok = nk > 0 && mbar_wait(bar_done, 0, p.status, where | 3);
    tc_fence_after();
    __syncthreads();
    const uint32_t trow = tmem + (static_cast<uint32_t>(warp * 32) << 16);
    const int row = tid, n = n0 + row;

    // The code below runs once per CTA, straight from a cold instruction cache: rolled loops over groups of 8
    // tokens (one tensor-memory round trip per group, not per token: with 256 tokens the round trips were a
    // third of the kernel).  Tokens are owned in contiguous blocks of red_rows: CTA r finishes tokens
    // [r * red_rows, (r + 1) * red_rows).
    const int t_lo = rank * p.red_rows, t_hi = min(p.M, t_lo + p.red_rows);
    if (S > 1) {
        if (ok) {
#pragma unroll 1
            for (int t0 = 0; t0 < p.M; t0 += 8) {
                if (t0 >= t_lo && t0 + 8 <= t_lo + p.red_rows) continue;  // all mine
                uint32_t v[8];
                tmem_ld8(trow + t0, v);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int t = t0 + i, owner = t / p.red_rows;
                    if (t >= p.M || owner == rank) continue;
                    const int slot = (rank - owner - 1 + S) % S;
                    const uint32_t local = red_base + ((slot * p.red_rows + (t - owner * p.red_rows)) * 128 + row) * 4;
                    dsmem_st_f32(dsmem_addr(local, owner), __uint_as_float(v[i]));
                }
            }
        }
        cluster_sync_all();  // every thread of every CTA, also after a failed wait
    }

    if (ok) {
        const float nw = (p.next_norm_w != nullptr && n < p.N) ? 1.0f + __bfloat162float(p.next_norm_w[n]) : 1.0f;
#pragma unroll 1
        for (int t0 = t_lo & ~7; t0 < t_hi; t0 += 8) {
            // the group's residual values are requested together, before anything waits for one of them
            float rv[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int t = t0 + i;
                rv[i] = (p.resid != nullptr && n < p.N && t >= t_lo && t < t_hi) ? __ldcg(p.resid + static_cast<size_t>(t) * p.ldr + n) : 0.0f;
            }
            uint32_t v[8];
            tmem_ld8(trow + t0, v);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int t = t0 + i;
                if (t < t_lo || t >= t_hi) continue;  // uniform over the CTA
                float acc = __uint_as_float(v[i]);
#pragma unroll 1
                for (int src = 0; src < S - 1; ++src) acc += red[(src * p.red_rows + (t - t_lo)) * 128 + row];
                acc *= rs[t];
                if (n < p.N) {
                    acc += rv[i];
                    if (p.out != nullptr) {
                        if (p.out_fp32) static_cast<float*>(p.out)[static_cast<size_t>(t) * p.ldo + n] = acc;
                        else static_cast<__nv_bfloat16*>(p.out)[static_cast<size_t>(t) * p.ldo + n] = __float2bfloat16(acc);
                    }
                    if (p.out_normed != nullptr) {
                        if (p.normed_fp16)
                            reinterpret_cast<__half*>(p.out_normed)[static_cast<size_t>(t) * p.ldn + n] =
                                __float2half_rn(fminf(fmaxf(acc * nw, -65504.0f), 65504.0f));
                        else
                            p.out_normed[static_cast<size_t>(t) * p.ldn + n] = __float2bfloat16(acc * nw);
                    }
                } else {
                    acc = 0.0f;
                }
                if (p.out_ssq != nullptr) {
                    const float q = warp_sum(acc * acc);
                    if (lane == 0) wsum[warp][t] = q;
                }
            }
        }
        if (p.out_ssq != nullptr) {
            __syncthreads();
            for (int t = t_lo + tid; t < t_hi; t += 128)
                p.out_ssq[blockIdx.y * p.M + t] = (wsum[0][t] + wsum[1][t]) + (wsum[2][t] + wsum[3][t]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, p.tmem_cols);
}

}  // namespace msk

extern "C" int msk_proj_skinny(const MskProjParams* q, int* status, void* stream) {
    using namespace msk;
    if (q == nullptr || q->x == nullptr || q->w == nullptr) return MSK_ERR_INVALID;
    if (q->M < 1 || q->M > 256 || q->N < 1 || q->K < 64 || q->K % 64 != 0) return MSK_ERR_UNSUPPORTED;
    if (q->out == nullptr && q->out_normed == nullptr) return MSK_ERR_INVALID;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) != cudaSuccess) return MSK_ERR_CUDA;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int tiles = (q->N + 127) / 128, KT = q->K / 64;
    int S = q->splits;
    if (S <= 0) {
        // a power of two: clusters of 3, 5, 6 or 7 CTAs leave SMs unused (they cannot span GPCs)
        S = 1;
        while (2 * S * tiles <= sms && S < 8) S *= 2;
    }
    if (S > 8) return MSK_ERR_UNSUPPORTED;
    if (S > KT) S = KT;
    const int bn = (q->M + 15) / 16 * 16;
    uint32_t cols = 32;
    while (cols < static_cast<uint32_t>(bn)) cols *= 2;
    const int red_rows = (bn + S - 1) / S;
    const int red_bytes = S > 1 ? (S - 1) * red_rows * 128 * 4 : 0;
    const int stage = kProjWBytes + bn * 128;
    const int budget = 232448 - 7168 - 1024 - red_bytes;  // opt-in limit minus static shared memory and alignment slack
    int nst = budget / stage;
    if (nst > kProjMaxStages) nst = kProjMaxStages;
    const int per_cta = (KT + S - 1) / S;
    if (nst > per_cta) nst = per_cta;
    if (nst < 2 && per_cta >= 2) return MSK_ERR_UNSUPPORTED;
    const int smem = 1024 + nst * stage + red_bytes;

    CUtensorMap tm_w, tm_x;
    int rc = make_tmap_bf16_2d(&tm_w, q->w, q->N, q->K, q->K, 128);
    if (rc == 0) rc = make_tmap_bf16_2d(&tm_x, q->x, q->M, q->K, q->K, bn);
    if (rc != 0) return rc;

    ProjArgs a{};
    a.M = q->M, a.N = q->N, a.K = q->K, a.bn = bn, a.nstages = nst, a.red_rows = red_rows, a.tmem_cols = cols;
    a.out = q->out, a.out_fp32 = q->out_fp32, a.ldo = q->ldo;
    a.in_ssq = q->in_ssq, a.in_ssq_parts = q->in_ssq_parts, a.in_inv_dim = q->in_inv_dim, a.in_eps = q->in_eps;
    a.resid = q->resid, a.ldr = q->ldr;
    a.next_norm_w = static_cast<const __nv_bfloat16*>(q->next_norm_w);
    a.out_normed = static_cast<__nv_bfloat16*>(q->out_normed), a.ldn = q->ldn, a.normed_fp16 = q->normed_fp16;
    a.out_ssq = q->out_ssq, a.status = status;

    static int configured_smem = 0;
    if (smem > configured_smem) {
        if (cudaFuncSetAttribute(proj_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return MSK_ERR_CUDA;
        configured_smem = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(S, tiles, 1);
    cfg.blockDim = dim3(128, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attrs[2];
    int na = 0;
    attrs[na].id = cudaLaunchAttributeClusterDimension;
    attrs[na].val.clusterDim.x = S;
    attrs[na].val.clusterDim.y = 1;
    attrs[na].val.clusterDim.z = 1;
    ++na;
    if (q->pdl) {
        attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = na;
    cudaError_t e = cudaLaunchKernelEx(&cfg, proj_skinny_kernel, tm_w, tm_x, a);
    return e == cudaSuccess ? 0 : MSK_ERR_CUDA;
}

// Tuning aid: how many clusters of `splits` CTAs with `smem_bytes` of dynamic shared memory the device
// can keep resident at once (cudaOccupancyMaxActiveClusters).  Negative on error.
extern "C" int msk_proj_max_active_clusters(int splits, int smem_bytes) {
    using namespace msk;
    if (splits < 1 || splits > 8 || smem_bytes < 0) return MSK_ERR_INVALID;
    if (cudaFuncSetAttribute(proj_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess)
        return MSK_ERR_CUDA;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(splits, 148, 1);
    cfg.blockDim = dim3(128, 1, 1);
    cfg.dynamicSmemBytes = smem_bytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, proj_skinny_kernel, &cfg) != cudaSuccess) return MSK_ERR_CUDA;
    return n;
}

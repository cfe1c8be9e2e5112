// Gated attention decode (L = 1) and 8-token verify (L = 8) over a paged FP8-E4M3 KV cache, one launch.
//
// Grid (chunks C, KV heads, requests); the C CTAs of one (request, KV head) form a thread block
// cluster and split that request's cached keys between them (split-KV).
// Decode CTA: 320 threads = eight arithmetic warps (two row groups of four: one warp per 32-key quarter of a tile,
// a row group per four query rows), one MMA warp and one copying warp, two CTAs per SM; verify CTA: 576 threads =
// sixteen arithmetic warps (four row groups of 16 rows) and the same two, one CTA per SM.  The two extra warps do
// nothing but issue (both MMAs of every tile / the TMA copies) and meet the others only through mbarriers; the K
// half and the V half of a ring slot are refilled the moment the MMA that read them has finished, so each copy has
// about two tiles' time to land; score buffers, P and the output accumulator are double-buffered, so a tile's
// second MMA has a whole iteration before its result is folded in; the arithmetic warps are left with one (decode)
// or two (verify) named barriers per tile, each over the four warps of a row group.
// (Timestamps showed why: with two arithmetic warps issuing, a decode tile cost 4200 clocks per CTA, 1200 of them
// the wait for a copy that had been issued a moment before it was needed and 1400 the issuing itself, on the path
// of all eight warps; now 2200, against 2900 for two CTAs per SM at the copy bandwidth.  Verify is bound by the
// arithmetic warps' instruction issue: ~25 instructions per (key, row) element.)
//
// Per 128-key tile (two 64-token pages, or 128 / page_size pages):
//   TMA      4-D boxes [page_size tokens x 128 B] of K and of V land in shared memory with the
//            128-byte swizzle; the physical page id from the block table is a runtime coordinate.
//   MMA 1    S^T[key, row] = K[key, :] . Q[row, :]   tcgen05.mma kind::f8f6f4, M = 128 keys,
//            N = 8 L query rows (row = 8 * token + head-in-group), K = head_dim 128.
//            The FP8 cache bytes are the A operand as they are (exact, no conversion); the query,
//            rounded to BF16 like the reference, is split into two E4M3 terms q = hi + lo
//            stacked as 2 x 8 L rows of one B tile (the second term times 16, its columns are scaled back when
//            read), which keeps BF16-level precision on FP8 tensor cores with a single pass over K.
//   softmax  thread = key: tcgen05.ld its row of S^T, scale, window / causal mask, running maximum
//            per query row (redux.sync over the warp, shared memory over the 4 warps), p = 2^(s-m)
//            split into two E4M3 terms the same way, written as the K-major B operand P[row, key].
//   MMA 2    O^T[d, row] = V^T[d, key] . P[row, key]; V stays as stored (MN-major A operand).
//   acc      thread = d: o[row] = o[row] * alpha[row] + O^T[d, row]  (FP32 registers).
// The L new tokens never travel through global memory: the last CTA of the cluster applies
// RMSNorm + RoPE to the new keys, quantises keys and values to E4M3, writes them to the cache
// rows `cache_loc` and attends them from registers / shared memory in FP32 (decode: before the tile loop, with
// the loads of the query rows, so that nothing but the fold-in is left for the end; verify: after the loop).
// Verify blocks (64 query rows per KV head) run the same tile loop with four row groups of 16 rows, each a full set
// of four warps (one per 32-key quarter of the tile), so that a thread's serial work per tile is 16 rows and several
// warps share every scheduler (with one warp per scheduler the 64-row loop ran ten times longer per tile than
// decode's 8 rows).
// Merge: every CTA pushes its (m, l, o) partials for the query rows another CTA owns into that
// CTA's shared memory (DSMEM), one cluster barrier, then each owner merges, applies the per-head
// RMSNorm and the sigmoid gate and stores BF16.
// Roofline: HBM (K and V bytes of the visible keys, read once).
#include <cuda_fp8.h>

#include "msk.h"
#include "ptx.cuh"
#include "tmap.cuh"

namespace msk {

constexpr int kAttnMaxStages = 6;
constexpr int kTileKeys = 128;
constexpr int kStageBytes = 2 * kTileKeys * 128;  // K tile + V tile
constexpr int kMaxTilesPerCta = 160;
constexpr float kNeg = -1.0e30f;
constexpr float kPScale = 256.0f;  // p in [0, 1] is stored as p * 256 (E4M3 / E5M2 range)

struct AttnArgs {
    const __nv_bfloat16* qkv;
    int ld_qkv;
    __nv_bfloat16* out;
    int ld_out;
    uint8_t* k_cache;
    uint8_t* v_cache;
    const float* k_scale;
    const float* v_scale;
    const int* seq_lens;
    const int* page_table;
    int max_pages;
    const long long* cache_loc;
    const float* inv_freq;
    int B, Hq, Hkv, page_size, num_pages, window, nstages, longest_first;
    float qk_scale_factor, sm_scale, q_split_scale;
    int* status;
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float redux_max(float v) {
    float r;
    asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
    return r;
}
__device__ __forceinline__ uint32_t f2_to_e4m3x2(float a, float b) {
    return __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ float e4m3_to_f(uint32_t byte) {
    __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(byte), __NV_E4M3);
    return __half2float(*reinterpret_cast<__half*>(&h));
}
__device__ __forceinline__ float2 e4m3x2_to_f2(uint32_t two) {  // low byte -> x
    __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(two), __NV_E4M3);
    return __half22float2(*reinterpret_cast<__half2*>(&h));
}
__device__ __forceinline__ uint32_t f_to_e4m3(float a) {
    return __nv_cvt_float_to_fp8(a, __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ uint32_t f_to_e5m2(float a) {
    return __nv_cvt_float_to_fp8(a, __NV_SATFINITE, __NV_E5M2);
}

// RMSNorm (weightless, eps 1e-5) and interleaved RoPE of one 128-wide head row held 4 values per lane.
__device__ __forceinline__ void norm_rope_row(float (&x)[4], float post_scale, const float* inv_freq, int pos, int lane) {
    float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss * (1.0f / 128.0f) + 1e-5f);
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] = (x[i] * r) * post_scale;
    if (inv_freq != nullptr) {
        const float fp = static_cast<float>(pos);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float ang = fp * inv_freq[2 * lane + h];
            const float c = cosf(ang), s = sinf(ang);
            const float e = x[2 * h], o = x[2 * h + 1];
            x[2 * h] = e * c - o * s;
            x[2 * h + 1] = e * s + o * c;
        }
    }
}

// TMEM load of BR (4 or 8) consecutive 32-bit columns
template <int BR>
__device__ __forceinline__ void tmem_ld_rows(uint32_t taddr, uint32_t (&r)[BR]) {
    if constexpr (BR == 8) tmem_ld8(taddr, r);
    else tmem_ld4(taddr, r);
}

// L: tokens per request (1 decode, 8 verify); RG: row groups = sets of four arithmetic warps (one warp per 32-key
// quarter of a tile) that split the 8 L query rows.  Two more warps do nothing but issue -- one the TMA copies, one
// both MMAs of every tile -- and meet the others only through mbarriers; score buffers, P tiles and output
// accumulators are double-buffered, so a tile's second MMA has a whole iteration before its result is folded in.
__host__ __device__ constexpr uint32_t attn_tmem_cols(int L) {  // two score and two output buffers of 16 L columns
    return 64 * L <= 64 ? 64 : 64 * L <= 128 ? 128 : 64 * L <= 256 ? 256 : 512;
}

template <int L, int RG>
__global__ void __launch_bounds__(128 * RG + 64, (L == 1 && RG <= 2) ? 2 : 1)
    attn_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, AttnArgs p) {
    constexpr int NR = 8 * L;                 // query rows per KV head
    constexpr int NTHR_C = 128 * RG, NWARP_C = NTHR_C / 32;  // arithmetic threads / warps
    constexpr int NTHR = NTHR_C + 64, NWARP = NTHR / 32;  // + the MMA warp and the copying warp
    constexpr int NRG = NR / RG;              // query rows per row group: a thread's serial work per tile
    constexpr int BR = NRG < 8 ? NRG : 8;     // rows per tensor-memory round trip
    static_assert(NRG % BR == 0 && (BR == 4 || BR == 8), "row groups work on blocks of 4 or 8 rows");
    constexpr int NP = 2 * NR;                // UMMA N: rows [0, NR) hold the first split term, [NR, 2 NR) the second
    constexpr int SBUF = 2;                   // score buffers in TMEM: the next tile's scores are computed ahead
    constexpr int PBUF = 2;                   // P tiles in shared memory and output accumulators in TMEM
    // SBUF * NP score columns, then PBUF * NP output columns, as a power of two
    constexpr uint32_t kCols = attn_tmem_cols(L);
    static_assert((SBUF + PBUF) * NP <= kCols, "tensor-memory columns");
    constexpr uint32_t kOCol = SBUF * NP;
    constexpr int QP_BYTES = NP * 128;
    constexpr float kLoScale = 16.0f;         // the second split term is stored times 16 (keeps small residuals in range)

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[4 * kAttnMaxStages + 2];
    __shared__ uint32_t tmem_slot;
    __shared__ int page_ids[kMaxTilesPerCta * 2];
    __shared__ __align__(16) float wred_s[PBUF][4][NR];  // per-warp maxima of a tile (alternating buffers)
    auto& wred = wred_s[0];
    __shared__ float m_s[NR], alpha_s[PBUF][NR], mrg_m[NR], mrg_l[NR];
    __shared__ float sc_tail[NR][L];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kq = warp & 3, rg = warp >> 2;  // 32-key quarter of the tile (= tensor-memory lane quarter), row group
    const int ktid = tid & 127;               // key inside the tile / channel d, depending on the phase
    const int r_lo = rg * NRG;                // this thread's query rows: [r_lo, r_lo + NRG)
    const int C = gridDim.x, rank = blockIdx.x, h = blockIdx.y;
    int b = blockIdx.z;
    if (p.longest_first) {
        // More CTAs than the GPU holds at once, contexts of very different lengths: the CTAs are handed out in
        // grid order, so slice z takes the request with the z-th longest context and the last wave is made of
        // short requests (list scheduling, longest first).  Every CTA ranks the <= 256 lengths itself.
        __shared__ int lens_s[256];
        __shared__ int b_s;
        for (int i = threadIdx.x; i < p.B; i += NTHR) lens_s[i] = p.seq_lens[i];
        __syncthreads();
        for (int j = threadIdx.x; j < p.B; j += NTHR) {
            const int lj = lens_s[j];
            int r = 0;
            for (int i = 0; i < p.B; ++i) {
                const int li = lens_s[i];
                r += (li > lj || (li == lj && i < j)) ? 1 : 0;
            }
            if (r == static_cast<int>(blockIdx.z)) b_s = j;
        }
        __syncthreads();
        b = b_s;
    }
    const int where = MSK_K_ATTN << 8;
    const int nst = p.nstages;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t s_q = base + nst * kStageBytes, s_p = s_q + QP_BYTES, s_mrg = s_p + PBUF * QP_BYTES;
    uint8_t* g_q = gbase + nst * kStageBytes;
    uint8_t* g_p = g_q + QP_BYTES;
    float* mrg_o = reinterpret_cast<float*>(g_q + (1 + PBUF) * QP_BYTES);  // [NR][128]
    // Barriers.  The K half and the V half of a ring slot fill and drain on their own (full / full_v); "scores exist"
    // (sdone) and "output product exists" (odone) are kept per ring slot, because the copying warp waits on them too,
    // to refill the half they free: a barrier per slot cannot complete twice before that warp has looked, since the
    // next tile of the slot needs the refill itself.
    auto full = [&](int s) { return smem_u32(&bars[s]); };
    auto full_v = [&](int s) { return smem_u32(&bars[kAttnMaxStages + s]); };
    auto sdone = [&](int s) { return smem_u32(&bars[2 * kAttnMaxStages + s]); };
    auto odone = [&](int s) { return smem_u32(&bars[3 * kAttnMaxStages + s]); };
    auto pready = [&](int i) { return smem_u32(&bars[4 * kAttnMaxStages + (i & 1)]); };  // P of tile i written

    // ---------------- set-up that does not depend on the previous kernel
    if (warp == 0) {
        tmem_alloc(smem_u32(&tmem_slot), kCols);
        tmem_relinquish();
    }
    if (tid == NTHR_C + 32) {  // the copying thread, which goes on to start the first copies itself
        for (int s = 0; s < nst; ++s) mbar_init(full(s), 1), mbar_init(full_v(s), 1), mbar_init(sdone(s), 1), mbar_init(odone(s), 1);
        mbar_init(pready(0), NWARP_C);
        mbar_init(pready(1), NWARP_C);
        fence_mbar_init();
    }
    const int seq = p.seq_lens[b];
    const int W = p.window;
    const int lo_all = W > 0 ? max(0, seq - W + 1) : 0;
    const int tiles_total = seq > 0 ? ((seq - 1) / kTileKeys - lo_all / kTileKeys + 1) : 0;
    const int t_first = lo_all / kTileKeys;
    const int per = (tiles_total + C - 1) / C;
    const int t_begin = t_first + rank * per;
    int nt = min(per, t_first + tiles_total - t_begin);
    if (nt < 0) nt = 0;
    if (nt > kMaxTilesPerCta) {
        if (tid == 0) report(p.status, MSK_ERR_CAPACITY, where | 1, nt, kMaxTilesPerCta);
        nt = kMaxTilesPerCta;
    }
    const int ppt = kTileKeys / p.page_size;  // pages per tile
    // The copying warp only arrives at the CTA's first barrier (it made the mbarriers, the others wait for them
    // there) and takes no part in the fills below; its thread fetches the page ids of the first tile itself and
    // starts that copy at once instead of waiting for the shared table.
    constexpr int NTHR_F = NTHR_C + 32;  // threads that fill shared memory before the first barrier
    int started = 0;                     // tiles whose copies are under way
    {
        if (warp == NWARP_C + 1) {
            __syncwarp();
            named_bar_arrive<4>(NTHR);
            if (lane == 0 && nt > 0 && ppt <= 8) {
                prefetch_tmap(&tm_k);
                prefetch_tmap(&tm_v);
                int ids[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const int pg = t_begin * ppt + k;
                    int id = (k < ppt && pg < p.max_pages) ? p.page_table[b * p.max_pages + pg] : -1;
                    if (id >= p.num_pages || id < -1) id = -1;  // reported by the table fill below
                    ids[k] = id;
                }
                mbar_expect_tx(full(0), kTileKeys * 128);
                mbar_expect_tx(full_v(0), kTileKeys * 128);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    if (k < ppt) {
                        tma_load_4d(base + k * p.page_size * 128, &tm_k, full(0), 0, h, 0, ids[k]);
                        tma_load_4d(base + kTileKeys * 128 + k * p.page_size * 128, &tm_v, full_v(0), 0, h, 0, ids[k]);
                    }
                }
                started = 1;
            }
        }
    }
    for (int i = tid; i < nt * ppt && tid < NTHR_F; i += NTHR_F) {
        const int pg = t_begin * ppt + i;
        int id = pg < p.max_pages ? p.page_table[b * p.max_pages + pg] : -1;
        if (id >= p.num_pages || id < -1) {
            report(p.status, MSK_ERR_BOUNDS, where | 2, id, p.num_pages);
            id = -1;
        }
        page_ids[i] = id;
    }
    for (int i = tid; i < (1 + PBUF) * QP_BYTES / 16 && tid < NTHR_F; i += NTHR_F)
        reinterpret_cast<uint4*>(g_q)[i] = make_uint4(0, 0, 0, 0);
    if (tid < NR) m_s[tid] = kNeg;
    tc_fence_before();
    // barrier 5: the table and the zeroed operands exist (the copying warp waits for this one, the others only
    // arrive); barrier 4: the mbarriers and the tensor-memory address exist (the other way round)
    if (warp == NWARP_C + 1) {
        named_bar_sync<5>(NTHR);
    } else {
        named_bar_arrive<5>(NTHR);
        named_bar_sync<4>(NTHR);
    }
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    pdl_launch_dependents();

    auto issue_half = [&](int i, int s, bool values) {  // one thread: the keys or the values of tile i into their half of slot s
        const uint32_t dst = base + s * kStageBytes + (values ? kTileKeys * 128 : 0);
        const uint32_t bar = values ? full_v(s) : full(s);
        mbar_expect_tx(bar, kTileKeys * 128);
        for (int j = 0; j < ppt; ++j)
            tma_load_4d(dst + j * p.page_size * 128, values ? &tm_v : &tm_k, bar, 0, h, 0, page_ids[i * ppt + j]);
    };
    // `slot`: ring slot of tile i (i % nst; the roles count it instead of dividing)
    auto issue_mma1 = [&](int i, int slot, uint32_t done) {  // S^T = K . q^T into score buffer i & 1
        const uint32_t kb = base + slot * kStageBytes;
        const uint32_t idesc = umma_idesc(128, NP, 0, 0, 0, 0);
        const uint64_t ad = umma_smem_desc(kb, 16, 1024, kSwizzle128);
        const uint64_t bq = umma_smem_desc(s_q, 16, 1024, kSwizzle128);
        const uint32_t d = tmem + (i & 1) * NP;
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_f8_ss(d, ad + 2 * k, bq + 2 * k, idesc, k != 0);
        umma_commit(done);
    };
    auto issue_mma2 = [&](int i, int slot, uint32_t done) {  // O^T = V^T . P^T from P buffer i & 1 into output buffer i & 1
        const uint32_t vb = base + slot * kStageBytes + kTileKeys * 128;
        const uint32_t idesc = umma_idesc(128, NP, 0, 0, 1, 0);
        const uint64_t bp = umma_smem_desc(s_p + (i & 1) * QP_BYTES, 16, 1024, kSwizzle128);
        const uint32_t d = tmem + kOCol + (i & 1) * NP;
        const uint64_t av = umma_smem_desc(vb, 1024, 1024, kSwizzle128);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_f8_ss(d, av + (4096 >> 4) * k, bp + 2 * k, idesc, k != 0);
        umma_commit(done);
    };

    if (tid == NTHR_C + 32) {
        if (started == 0) {
            prefetch_tmap(&tm_k);
            prefetch_tmap(&tm_v);
        }
        for (int i = started; i < nt && i < nst; ++i) {
            issue_half(i, i, false);
            issue_half(i, i, true);
        }
    }

    // ---------------- queries: RMSNorm, scale, RoPE, BF16 rounding, split into two E4M3 terms
    pdl_wait();
    const float k_scale = __ldg(p.k_scale), v_scale = __ldg(p.v_scale);
    const float qs = p.q_split_scale;
    // Decode: the new token's part of the step needs nothing from the cache, so the cluster's last CTA does it here,
    // with the loads in flight together: every warp derives the new key itself (registers only) and takes the
    // score of its query row against it; warp 0 also stores the new key and value bytes; each arithmetic thread
    // keeps the new value of its channel and the gates of the rows it will finalise.
    const bool tail_cta = rank == C - 1;
    float vnew_d = 0.0f;
    float gate_r[L == 1 ? NRG : 1];
    if constexpr (L == 1) {
        const int rows_per_cta = NR / C;
#pragma unroll
        for (int k = 0; k < NRG; ++k) {
            const int nl = rg + k * RG, n = rank * rows_per_cta + nl;
            gate_r[k] = (warp < NWARP_C && nl < rows_per_cta)
                            ? __bfloat162float(p.qkv[static_cast<size_t>(b) * p.ld_qkv + (p.Hq + 2 * p.Hkv + h * 8 + (n & 7)) * 128 + ktid])
                            : 0.0f;
        }
        if (tail_cta && warp < NWARP_C) {
            const float v = __bfloat162float(p.qkv[static_cast<size_t>(b) * p.ld_qkv + (p.Hq + p.Hkv + h) * 128 + ktid]);
            vnew_d = e4m3_to_f(f_to_e4m3(__fdiv_rn(v, v_scale)));
        }
    }
    for (int n = warp; n < NR; n += NWARP) {
        const int j = n >> 3, g = n & 7;
        const size_t tok = static_cast<size_t>(b) * L + j;
        const __nv_bfloat16* src = p.qkv + tok * p.ld_qkv + (h * 8 + g) * 128 + 4 * lane;
        const uint2 raw = *reinterpret_cast<const uint2*>(src);
        float x[4] = {bf16lo(raw.x), bf16hi(raw.x), bf16lo(raw.y), bf16hi(raw.y)};
        float knew_r[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (L == 1 && tail_cta) {
            const __nv_bfloat16* ksrc = p.qkv + tok * p.ld_qkv + (p.Hq + h) * 128 + 4 * lane;
            const uint2 kr = *reinterpret_cast<const uint2*>(ksrc);
            uint2 vr = make_uint2(0, 0);
            long long row = -1;
            if (n == 0) {
                vr = *reinterpret_cast<const uint2*>(ksrc + p.Hkv * 128);
                row = p.cache_loc[tok];
            }
            float kx[4] = {bf16lo(kr.x), bf16hi(kr.x), bf16lo(kr.y), bf16hi(kr.y)};
            norm_rope_row(kx, 1.0f, p.inv_freq, seq, lane);
            uint32_t kb = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t a = f_to_e4m3(__fdiv_rn(kx[i], k_scale));
                kb |= a << (8 * i);
                knew_r[i] = e4m3_to_f(a);
            }
            if (n == 0) {
                const float vx[4] = {bf16lo(vr.x), bf16hi(vr.x), bf16lo(vr.y), bf16hi(vr.y)};
                uint32_t vb = 0;
#pragma unroll
                for (int i = 0; i < 4; ++i) vb |= f_to_e4m3(__fdiv_rn(vx[i], v_scale)) << (8 * i);
                const bool row_ok = row >= 0 && row < static_cast<long long>(p.num_pages) * p.page_size;
                if (!row_ok && lane == 0) report(p.status, MSK_ERR_BOUNDS, where | 7, static_cast<int>(row), p.num_pages);
                if (row_ok) {
                    const size_t off = (static_cast<size_t>(row) * p.Hkv + h) * 128 + 4 * lane;
                    *reinterpret_cast<uint32_t*>(p.k_cache + off) = kb;
                    *reinterpret_cast<uint32_t*>(p.v_cache + off) = vb;
                }
            }
        }
        norm_rope_row(x, p.qk_scale_factor, p.inv_freq, seq + j, lane);
        if (L == 1 && tail_cta) {
            float dot = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) dot += __bfloat162float(__float2bfloat16(x[i])) * knew_r[i];
            dot = warp_sum(dot);
            if (lane == 0) sc_tail[n][0] = dot * (k_scale * p.sm_scale * 1.4426950408889634f);
        }
        uint32_t hi = 0, lo = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float q = __bfloat162float(__float2bfloat16(x[i])) * qs;
            const uint32_t bh = f_to_e4m3(q);
            const uint32_t bl = f_to_e4m3((q - e4m3_to_f(bh)) * kLoScale);
            hi |= bh << (8 * i);
            lo |= bl << (8 * i);
        }
        *reinterpret_cast<uint32_t*>(g_q + swz128(n, 4 * lane)) = hi;
        *reinterpret_cast<uint32_t*>(g_q + swz128(NR + n, 4 * lane)) = lo;
    }
    fence_proxy_async_smem();
    __syncthreads();

    // ---------------- main loop over this CTA's cached tiles
    float l_part[NRG], o_acc[NRG];  // of rows r_lo + n
#pragma unroll
    for (int n = 0; n < NRG; ++n) l_part[n] = 0.0f, o_acc[n] = 0.0f;
    const float s_scale = k_scale * p.sm_scale * 1.4426950408889634f / qs;
    const uint32_t trow = tmem + (static_cast<uint32_t>(kq * 32) << 16);
    bool ok = true;
    // decode keeps the running maxima and the rescale factors replicated in every thread's registers
    float m_r[L == 1 ? NRG : 1], alpha_r[L == 1 ? NRG : 1];  // of rows r_lo + g
#pragma unroll
    for (int g = 0; g < (L == 1 ? NRG : 1); ++g) m_r[g] = kNeg, alpha_r[g] = 1.0f;

    // scores of BR query rows (c0 .. c0+BR-1) for this thread's key: both split terms
    auto load_scores = [&](int i, int c0, float (&sc)[BR]) {
        uint32_t hi[BR], lo[BR];
        const uint32_t col = trow + (i & 1) * NP + c0;
        tmem_ld_rows<BR>(col, hi);
        tmem_ld_rows<BR>(col + NR, lo);
        tmem_wait_ld();
#pragma unroll
        for (int g = 0; g < BR; ++g) sc[g] = __uint_as_float(hi[g]) + __uint_as_float(lo[g]) * (1.0f / kLoScale);
    };
    // second half of a tile's work: wait for O^T = V^T . P^T (output buffer j & 1) and fold it into the running
    // output with tile j's rescale factors (decode: `al_j`).  It runs at the end of the next iteration, so the MMA
    // has had a whole iteration to finish.
    auto finish_tile = [&](int j, const float* al_j, uint32_t done, int parity) {
        ok = mbar_wait(done, parity, p.status, where | 6) && ok;
        tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < NRG; c0 += BR) {
            uint32_t hi[BR], lo[BR];
            const uint32_t col = trow + kOCol + (j & 1) * NP + r_lo + c0;
            tmem_ld_rows<BR>(col, hi);
            tmem_ld_rows<BR>(col + NR, lo);
            tmem_wait_ld();
#pragma unroll
            for (int g = 0; g < BR; ++g) {
                const float al = L == 1 ? al_j[c0 + g] : alpha_s[j & 1][r_lo + c0 + g];
                o_acc[c0 + g] = o_acc[c0 + g] * al + (__uint_as_float(hi[g]) + __uint_as_float(lo[g]) * (1.0f / kLoScale));
            }
        }
        tc_fence_before();
        __syncwarp();
    };

    {
      if (warp == NWARP_C) {
        // ---- the MMA warp: one thread, no arithmetic, no CTA barrier inside the loop
        if (lane == 0 && nt > 0) {
            bool live = mbar_wait(full(0), 0, p.status, where | 3);
            tc_fence_after();
            if (live) issue_mma1(0, 0, sdone(0));
            int s_cur = 0, ph_cur = 0;                               // ring slot and fill parity of tile i
            int s_nxt = nst > 1 ? 1 : 0, ph_nxt = nst > 1 ? 0 : 1;   // of tile i + 1
            for (int i = 0; i < nt && live; ++i) {
                if (i + 1 < nt) {  // the next tile's scores, one buffer ahead of their readers
                    live = mbar_wait(full(s_nxt), ph_nxt, p.status, where | 4);
                    tc_fence_after();
                    if (!live) break;
                    issue_mma1(i + 1, s_nxt, sdone(s_nxt));
                }
                live = mbar_wait(pready(i), (i >> 1) & 1, p.status, where | 8) &&
                       mbar_wait(full_v(s_cur), ph_cur, p.status, where | 9);
                if (!live) break;
                tc_fence_after();
                issue_mma2(i, s_cur, odone(s_cur));
                s_cur = s_nxt, ph_cur = ph_nxt;
                if (++s_nxt == nst) s_nxt = 0, ph_nxt ^= 1;
            }
        }
        __syncwarp();
      } else if (warp == NWARP_C + 1) {
        // ---- the copying warp: refills the K half of a slot as soon as its tile's scores exist and the V half as
        // soon as its output product exists; every copy then has about two iterations to land
        if (lane == 0) {
            int s_i = 0, ph_i = 0, s_p = 0, ph_p = 0;  // slot / parity of tile i and of tile i - 1
            for (int i = 0; i + nst < nt + 1; ++i) {
                if (i + nst < nt) {
                    if (!mbar_wait(sdone(s_i), ph_i, p.status, where | 10)) break;
                    issue_half(i + nst, s_i, false);
                }
                if (i >= 1) {
                    if (!mbar_wait(odone(s_p), ph_p, p.status, where | 11)) break;
                    issue_half(i - 1 + nst, s_p, true);
                }
                s_p = s_i, ph_p = ph_i;
                if (++s_i == nst) s_i = 0, ph_i ^= 1;
            }
        }
        __syncwarp();
      } else {
        // ---- the arithmetic warps.  Decode keeps the running maxima and rescale factors of its 4 rows in every
        // thread's registers (one named barrier per tile); verify keeps them in shared memory, written by one
        // thread per row of the row group between two named barriers.
        float alpha_p[L == 1 ? NRG : 1];  // decode: rescale factors of the tile before the current one (folded in late)
#pragma unroll
        for (int g = 0; g < (L == 1 ? NRG : 1); ++g) alpha_p[g] = 1.0f;
        auto rg_sync = [&]() {  // the four warps of this row group
            if (rg == 0) named_bar_sync<1>(128);
            else if (rg == 1) named_bar_sync<2>(128);
            else if (rg == 2) named_bar_sync<6>(128);
            else named_bar_sync<7>(128);
        };
        int slot = 0, ph = 0, slot_p = 0, ph_p = 0;  // ring slot / fill parity of tile i and of tile i - 1
        for (int i = 0; i < nt; ++i) {
            ok = mbar_wait(sdone(slot), ph, p.status, where | 5) && ok;
            tc_fence_after();
            const int pos = (t_begin + i) * kTileKeys + ktid;  // this thread's key position
            float skeep[NRG];
#pragma unroll
            for (int c0 = 0; c0 < NRG; c0 += BR) {
                float sc[BR];
                load_scores(i, r_lo + c0, sc);
                const int j = (r_lo + c0) >> 3;
                const bool vis = pos < seq && (W == 0 || pos > seq + j - W);
#pragma unroll
                for (int g = 0; g < BR; ++g) {
                    const float sv = vis ? sc[g] * s_scale : kNeg;
                    skeep[c0 + g] = sv;
                    const float mx = redux_max(sv);
                    if (lane == 0) wred_s[i & 1][kq][r_lo + c0 + g] = mx;
                }
            }
            rg_sync();  // the maxima buffers alternate, so decode needs no second barrier
            if constexpr (L == 1) {
                float tm[NRG];
#pragma unroll
                for (int w = 0; w < 4; ++w) {
#pragma unroll
                    for (int q4 = 0; q4 < NRG / 4; ++q4) {
                        const float4 a = *reinterpret_cast<const float4*>(&wred_s[i & 1][w][r_lo + 4 * q4]);
                        const float v4[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
                        for (int g = 0; g < 4; ++g) tm[4 * q4 + g] = w == 0 ? v4[g] : fmaxf(tm[4 * q4 + g], v4[g]);
                    }
                }
#pragma unroll
                for (int g = 0; g < NRG; ++g) {
                    const float mn = fmaxf(tm[g], m_r[g]);
                    alpha_p[g] = alpha_r[g];
                    alpha_r[g] = ex2(m_r[g] - mn);
                    m_r[g] = mn;
                }
            } else {
                if (ktid < NRG) {
                    const int r = r_lo + ktid;
                    const float mo = m_s[r];
                    const float mn = fmaxf(fmaxf(fmaxf(wred_s[i & 1][0][r], wred_s[i & 1][1][r]), fmaxf(wred_s[i & 1][2][r], wred_s[i & 1][3][r])), mo);
                    alpha_s[i & 1][r] = ex2(mo - mn);
                    m_s[r] = mn;
                }
            }
            // V rows past the cached length may hold anything (even NaN bytes): zero them so that 0 * V stays 0
            if (rg == 0 && pos >= seq) {
                ok = mbar_wait(full_v(slot), ph, p.status, where | 12) && ok;
                uint8_t* vrow = gbase + slot * kStageBytes + kTileKeys * 128 + ktid * 128;
#pragma unroll
                for (int c = 0; c < 8; ++c) reinterpret_cast<uint4*>(vrow)[c] = make_uint4(0, 0, 0, 0);
            }
            if constexpr (L != 1) rg_sync();
            // p = 2^(s - m) as two E4M3 terms into P buffer i & 1 (its previous reader, the second MMA of tile
            // i - 2, was waited for at the end of the last iteration)
            uint8_t* pb = g_p + (i & 1) * QP_BYTES;
#pragma unroll
            for (int g = 0; g < NRG; g += 2) {  // two rows per conversion instruction
                const int n = r_lo + g;
                const bool vis = pos < seq && (W == 0 || pos > seq + (n >> 3) - W);  // rows n and n + 1: same token
                const float m0 = L == 1 ? m_r[g] : m_s[n], m1 = L == 1 ? m_r[g + 1] : m_s[n + 1];
                const float a0 = L == 1 ? alpha_r[g] : alpha_s[i & 1][n], a1 = L == 1 ? alpha_r[g + 1] : alpha_s[i & 1][n + 1];
                const float pr0 = vis ? ex2(skeep[g] - m0) : 0.0f;
                const float pr1 = vis ? ex2(skeep[g + 1] - m1) : 0.0f;
                l_part[g] = l_part[g] * a0 + pr0;
                l_part[g + 1] = l_part[g + 1] * a1 + pr1;
                const float ps0 = pr0 * kPScale, ps1 = pr1 * kPScale;
                const uint32_t bh = f2_to_e4m3x2(ps0, ps1);
                const float2 back = e4m3x2_to_f2(bh);
                const uint32_t bl = f2_to_e4m3x2((ps0 - back.x) * kLoScale, (ps1 - back.y) * kLoScale);
                pb[swz128(n, ktid)] = static_cast<uint8_t>(bh);
                pb[swz128(n + 1, ktid)] = static_cast<uint8_t>(bh >> 8);
                pb[swz128(NR + n, ktid)] = static_cast<uint8_t>(bl);
                pb[swz128(NR + n + 1, ktid)] = static_cast<uint8_t>(bl >> 8);
            }
            tc_fence_before();
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(pready(i));
            if (i > 0) finish_tile(i - 1, alpha_p, odone(slot_p), ph_p);  // issued a whole iteration ago
            slot_p = slot, ph_p = ph;
            if (++slot == nst) slot = 0, ph ^= 1;
        }
        if (nt > 0) finish_tile(nt - 1, alpha_r, odone(slot_p), ph_p);
      }
    }
    // From here on the arithmetic threads only; the two issuing warps go straight to the cluster barrier.
    const int rows_per = NR / C;  // query rows each CTA finalises (C divides NR)
    auto csync = [&]() { named_bar_sync<3>(NTHR_C); };
    if (warp < NWARP_C) {
    if constexpr (L == 1) {
#pragma unroll
        for (int g = 0; g < NRG; ++g)
            if (ktid == g) m_s[r_lo + g] = m_r[g];
    }
    csync();

    // ---------------- the L new tokens: last CTA of the cluster, FP32 on CUDA cores
    // (decode: keys, values, cache rows and scores of the new token were done before the main loop)
    if (rank == C - 1) {
        float* knew = reinterpret_cast<float*>(gbase);                 // [L][128] E4M3 values of the new keys
        float* vnew = knew + L * 128;                                  // [L][128]
        __nv_bfloat16* qf = reinterpret_cast<__nv_bfloat16*>(vnew + L * 128);  // [NR][128] BF16 queries
        if constexpr (L != 1) {
        for (int j = warp; j < L; j += NWARP_C) {
            const size_t tok = static_cast<size_t>(b) * L + j;
            const long long row = p.cache_loc[tok];
            const bool row_ok = row >= 0 && row < static_cast<long long>(p.num_pages) * p.page_size;
            if (!row_ok && lane == 0) report(p.status, MSK_ERR_BOUNDS, where | 7, static_cast<int>(row), p.num_pages);
            const __nv_bfloat16* ksrc = p.qkv + tok * p.ld_qkv + (p.Hq + h) * 128 + 4 * lane;
            const __nv_bfloat16* vsrc = ksrc + p.Hkv * 128;
            const uint2 kr = *reinterpret_cast<const uint2*>(ksrc), vr = *reinterpret_cast<const uint2*>(vsrc);
            float kx[4] = {bf16lo(kr.x), bf16hi(kr.x), bf16lo(kr.y), bf16hi(kr.y)};
            const float vx[4] = {bf16lo(vr.x), bf16hi(vr.x), bf16lo(vr.y), bf16hi(vr.y)};
            norm_rope_row(kx, 1.0f, p.inv_freq, seq + j, lane);
            uint32_t kb = 0, vb = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t a = f_to_e4m3(__fdiv_rn(kx[i], k_scale)), c = f_to_e4m3(__fdiv_rn(vx[i], v_scale));
                kb |= a << (8 * i);
                vb |= c << (8 * i);
                knew[j * 128 + 4 * lane + i] = e4m3_to_f(a);
                vnew[j * 128 + 4 * lane + i] = e4m3_to_f(c);
            }
            if (row_ok) {
                const size_t off = (static_cast<size_t>(row) * p.Hkv + h) * 128 + 4 * lane;
                *reinterpret_cast<uint32_t*>(p.k_cache + off) = kb;
                *reinterpret_cast<uint32_t*>(p.v_cache + off) = vb;
            }
        }
        // BF16 queries again (the MMA operands hold them split)
        for (int n = warp; n < NR; n += NWARP_C) {
            const int j = n >> 3, g = n & 7;
            const size_t tok = static_cast<size_t>(b) * L + j;
            const uint2 raw = *reinterpret_cast<const uint2*>(p.qkv + tok * p.ld_qkv + (h * 8 + g) * 128 + 4 * lane);
            float x[4] = {bf16lo(raw.x), bf16hi(raw.x), bf16lo(raw.y), bf16hi(raw.y)};
            norm_rope_row(x, p.qk_scale_factor, p.inv_freq, seq + j, lane);
            *reinterpret_cast<uint2*>(qf + n * 128 + 4 * lane) = make_uint2(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]));
        }
        csync();
        // scores of (row n, new token r), r <= token of n (causal) and inside the window
        const float t_scale = k_scale * p.sm_scale * 1.4426950408889634f;
        for (int e = tid; e < NR * L; e += NTHR_C) {
            const int n = e / L, r = e % L, j = n >> 3;
            float acc = 0.0f;
            for (int d = 0; d < 128; d += 2) {
                const uint32_t qq = *reinterpret_cast<const uint32_t*>(qf + n * 128 + d);
                acc += bf16lo(qq) * knew[r * 128 + d] + bf16hi(qq) * knew[r * 128 + d + 1];
            }
            const bool vis = r <= j && (W == 0 || r > j - W);
            sc_tail[n][r] = vis ? acc * t_scale : kNeg;
        }
        csync();
        }
        if (tid < NR) {
            float mx = m_s[tid];
            const float mo = mx;
            for (int r = 0; r < L; ++r) mx = fmaxf(mx, sc_tail[tid][r]);
            alpha_s[0][tid] = ex2(mo - mx);
            m_s[tid] = mx;
        }
        csync();
#pragma unroll
        for (int n = 0; n < NRG; ++n) {
            const float a = alpha_s[0][r_lo + n], m = m_s[r_lo + n];
            float o = o_acc[n] * a;
            l_part[n] *= a;
#pragma unroll
            for (int r = 0; r < L; ++r) {
                const float sc = sc_tail[r_lo + n][r];
                const float pr = sc > 0.5f * kNeg ? ex2(sc - m) : 0.0f;
                o += pr * kPScale * (L == 1 ? vnew_d : vnew[r * 128 + ktid]);
                if (ktid == r) l_part[n] += pr;
            }
            o_acc[n] = o;
        }
    }

    // ---------------- merge across the cluster
#pragma unroll
    for (int n = 0; n < NRG; ++n) {
        const float s = warp_sum(l_part[n]);
        if (lane == 0) wred[kq][r_lo + n] = s;
    }
    csync();
    if (tid < NR) {
        const int owner = tid / rows_per, nl = tid % rows_per;
        const float lsum = (wred[0][tid] + wred[1][tid]) + (wred[2][tid] + wred[3][tid]);
        dsmem_st_f32(dsmem_addr(smem_u32(&mrg_m[rank * rows_per + nl]), owner), m_s[tid]);
        dsmem_st_f32(dsmem_addr(smem_u32(&mrg_l[rank * rows_per + nl]), owner), lsum);
    }
#pragma unroll
    for (int n = 0; n < NRG; ++n) {
        const int owner = (r_lo + n) / rows_per, nl = (r_lo + n) % rows_per;
        dsmem_st_f32(dsmem_addr(s_mrg + ((rank * rows_per + nl) * 128 + ktid) * 4, owner), o_acc[n]);
    }
    }
    cluster_sync_all();
    if (warp < NWARP_C) {

    // this CTA's rows nl = rg, rg + RG, ...: thread = channel d
    float val[NRG];
#pragma unroll
    for (int k = 0; k < NRG; ++k) {
        const int nl = rg + k * RG;
        if (nl >= rows_per) break;
        float mx = kNeg;
        for (int src = 0; src < C; ++src) mx = fmaxf(mx, mrg_m[src * rows_per + nl]);
        float lsum = 0.0f, o = 0.0f;
        for (int src = 0; src < C; ++src) {
            const float wgt = ex2(mrg_m[src * rows_per + nl] - mx);
            lsum += wgt * mrg_l[src * rows_per + nl];
            o += wgt * mrg_o[(src * rows_per + nl) * 128 + ktid];
        }
        const float vv = lsum > 0.0f ? o * (v_scale / kPScale) / lsum : 0.0f;
        val[k] = vv;
        const float ss = warp_sum(vv * vv);
        if (lane == 0) wred[kq][nl] = ss;
    }
    // the gates of this thread's rows are requested together (a load between two stores is not moved up by the
    // compiler, and one global round trip per row is most of this epilogue)
    // (decode asked for them before the main loop)
    float gate_l[L == 1 ? 1 : NRG];
    if constexpr (L != 1) {
#pragma unroll
        for (int k = 0; k < NRG; ++k) {
            const int nl = rg + k * RG, n = rank * rows_per + nl;
            const size_t tok = static_cast<size_t>(b) * L + (n >> 3);
            gate_l[k] = nl < rows_per ? __bfloat162float(p.qkv[tok * p.ld_qkv + (p.Hq + 2 * p.Hkv + h * 8 + (n & 7)) * 128 + ktid]) : 0.0f;
        }
    }
    csync();
    if (ok) {
#pragma unroll
        for (int k = 0; k < NRG; ++k) {
            const int nl = rg + k * RG;
            if (nl >= rows_per) break;
            const int n = rank * rows_per + nl, j = n >> 3, g = n & 7;
            const size_t tok = static_cast<size_t>(b) * L + j;
            const float ss = (wred[0][nl] + wred[1][nl]) + (wred[2][nl] + wred[3][nl]);
            const float r = 1.0f / sqrtf(ss * (1.0f / 128.0f) + 1e-5f);
            const float sg = 1.0f / (1.0f + __expf(-(L == 1 ? gate_r[k] : gate_l[k])));
            p.out[tok * p.ld_out + (h * 8 + g) * 128 + ktid] = __float2bfloat16(val[k] * r * sg);
        }
    }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kCols);
}

template <int L, int RG>
int launch_attn(const MskAttnParams* q, int* status, cudaStream_t stream) {
    constexpr int NR = 8 * L, NP = 2 * NR;
    constexpr int kColsHost = attn_tmem_cols(L);
    const int tile_cap = (q->max_pages * q->page_size + kTileKeys - 1) / kTileKeys;
    int tiles_max = tile_cap;
    if (q->window > 0) tiles_max = min(tiles_max, q->window / kTileKeys + 2);
    if (tiles_max < 1) tiles_max = 1;
    // the ring needs 3 slots: a tile's slot is refilled one iteration after its tile (finish_tile runs late),
    // and the next tile's scores are issued one iteration early
    if (q->stages != 0 && (q->stages < 3 || q->stages > kAttnMaxStages)) return MSK_ERR_INVALID;
    int nst = q->stages > 0 ? q->stages : 3;
    int smem = 1024 + nst * kStageBytes + 3 * NP * 128 + NR * 128 * 4;
    if (smem > 232448) return MSK_ERR_INVALID;
    int resident = min(232448 / (smem + 2048), 512 / kColsHost);  // CTAs per SM: shared memory, tensor memory
    if (resident < 1) resident = 1;
    int C = q->chunks;
    if (C <= 0) {
        int want = (resident * 148) / (q->B * q->Hkv);
        if (want > tiles_max) want = tiles_max;
        C = 1;
        while (2 * C <= want && C < 8) C *= 2;
        // more (request, head) pairs than CTA slots but fewer than two waves of them, and long contexts: halves
        // balance the last wave better; with several waves (longest first) whole contexts have less fixed cost
        if (C == 1 && tiles_max >= 32 && q->B * q->Hkv < 2 * resident * 148) C = 2;
        while ((tiles_max + C - 1) / C > kMaxTilesPerCta && C < 8) C *= 2;
    }
    if (C != 1 && C != 2 && C != 4 && C != 8) return MSK_ERR_INVALID;
    if ((tiles_max + C - 1) / C > kMaxTilesPerCta) return MSK_ERR_UNSUPPORTED;
    // The verify form is one CTA per SM whatever the ring: it takes the deepest that fits.  Decode stays at three
    // slots even when the grid is small: a deeper ring gained 0.3 us there and, being one CTA per SM, could not hold
    // 16 clusters of 8 at once (4 requests x 4 KV heads x 8 chunks took 28 us instead of 17).
    if (q->stages == 0 && L != 1) {
        const int fixed = 1024 + 3 * NP * 128 + NR * 128 * 4;
        nst = min(kAttnMaxStages, (232448 - fixed) / kStageBytes);
        smem = fixed + nst * kStageBytes;
    }

    CUtensorMap tm_k, tm_v;
    const uint64_t dims[4] = {128, static_cast<uint64_t>(q->Hkv), static_cast<uint64_t>(q->page_size),
                              static_cast<uint64_t>(q->num_pages)};
    const uint64_t strides[3] = {128, static_cast<uint64_t>(q->Hkv) * 128,
                                 static_cast<uint64_t>(q->Hkv) * 128 * q->page_size};
    const uint32_t box[4] = {128, 1, static_cast<uint32_t>(q->page_size), 1};
    int rc = make_tmap(&tm_k, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, q->k_cache, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc == 0)
        rc = make_tmap(&tm_v, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, q->v_cache, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != 0) return rc;

    AttnArgs a{};
    a.qkv = static_cast<const __nv_bfloat16*>(q->qkv), a.ld_qkv = q->ld_qkv;
    a.out = static_cast<__nv_bfloat16*>(q->out), a.ld_out = q->ld_out;
    a.k_cache = static_cast<uint8_t*>(q->k_cache), a.v_cache = static_cast<uint8_t*>(q->v_cache);
    a.k_scale = q->k_scale, a.v_scale = q->v_scale, a.seq_lens = q->seq_lens, a.page_table = q->page_table;
    a.max_pages = q->max_pages, a.cache_loc = reinterpret_cast<const long long*>(q->cache_loc), a.inv_freq = q->inv_freq;
    a.B = q->B, a.Hq = q->Hq, a.Hkv = q->Hkv, a.page_size = q->page_size, a.num_pages = q->num_pages;
    a.longest_first = (q->B <= 256 && q->B * q->Hkv * C > resident * 148) ? 1 : 0;
    a.window = q->window, a.nstages = nst, a.qk_scale_factor = q->qk_scale_factor, a.sm_scale = q->sm_scale;
    // largest power of two that keeps |q| * scale <= 448 (|q| <= qk_scale_factor * sqrt(128) after RMSNorm)
    float qs = 1.0f;
    const float qmax = fabsf(q->qk_scale_factor) * 11.3137085f;
    while (qs * 2.0f * qmax <= 448.0f && qs < 65536.0f) qs *= 2.0f;
    while (qs * qmax > 448.0f && qs > 1.0f / 65536.0f) qs *= 0.5f;
    a.q_split_scale = qs, a.status = status;

    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MSK_ERR_CUDA;
    static int configured[64] = {};  // per device, like the attribute itself
    if (smem > configured[dev]) {
        if (cudaFuncSetAttribute(attn_kernel<L, RG>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return MSK_ERR_CUDA;
        configured[dev] = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(C, q->Hkv, q->B);
    cfg.blockDim = dim3(128 * RG + 64, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    int na = 0;
    attrs[na].id = cudaLaunchAttributeClusterDimension;
    attrs[na].val.clusterDim.x = C;
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
    return cudaLaunchKernelEx(&cfg, attn_kernel<L, RG>, tm_k, tm_v, a) == cudaSuccess ? 0 : MSK_ERR_CUDA;
}

}  // namespace msk

extern "C" int msk_attn_decode(const MskAttnParams* q, int* status, void* stream) {
    using namespace msk;
    if (q == nullptr || !q->qkv || !q->out || !q->k_cache || !q->v_cache || !q->k_scale || !q->v_scale ||
        !q->seq_lens || !q->page_table || !q->cache_loc)
        return MSK_ERR_INVALID;
    if (q->d != 128 || q->Hkv < 1 || q->Hq != 8 * q->Hkv || q->B < 1) return MSK_ERR_UNSUPPORTED;
    if (q->page_size < 8 || q->page_size > 128 || (q->page_size & (q->page_size - 1)) != 0) return MSK_ERR_UNSUPPORTED;
    if (q->issuers != 0 && q->issuers != 1) return MSK_ERR_INVALID;
    if (q->row_groups != 0 && q->row_groups != (q->L == 1 ? 2 : 4)) return MSK_ERR_INVALID;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (q->L == 1) return launch_attn<1, 2>(q, status, s);  // 8 arithmetic warps + MMA warp + copying warp, 2 CTAs per SM
    if (q->L == 8) return launch_attn<8, 4>(q, status, s);  // 16 arithmetic warps + the same two
    return MSK_ERR_UNSUPPORTED;
}

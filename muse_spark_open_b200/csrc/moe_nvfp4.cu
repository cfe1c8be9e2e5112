// NVFP4 (w4a16) routed experts: grouped GEMMs with the routing done inside the GEMM CTAs.
//
//   stage    x16[row] = fp16(x[token(row)])   (only when x arrives as BF16, or for more than 32 tokens, where
//            the rows are also gathered into expert-list order)
//   gemm 1   h[pair, 2I] = x[token(pair)] . W13[expert(pair)]^T, and in its epilogue
//            inter[row, I] = fp16(silu(h_gate) * h_up), rows in expert-list order
//   gemm 2   y[pair, H]  = inter . W2[expert]^T
//   combine  out[t] = sum over the token's local (expert) slots of w[t, slot] * rmsnorm(y * (1 + w_post))
//
// A "pair" is one (token, routed slot).  Every gemm CTA rebuilds the routing in shared memory (from
// the given top-k ids, or from router logits: softmax, top-8, renormalise), turns it into per-expert
// pair lists and walks the work units (expert-group of <= 32 pairs, 128-row tile, K split) that fall
// to it, so every touched expert's weights stream through the SMs once.
//
// Arithmetic: FP16 x FP16 -> FP32 on the tensor cores.  Every E2M1 x E4M3 product (|v| in [2^-10, 2688], at
// most 5 significant bits) is exact in FP16, so the weights enter exactly; a BF16 activation converts to FP16
// exactly whenever 2^-14 <= |x| <= 65504 (8 significant bits into 11), smaller ones round to the 2^-24 grid
// (absolute error <= 2^-25 per element), larger ones saturate.  sm_100a converts two E2M1 codes to FP16x2 in
// one instruction (cvt.rn.f16x2.e2m1x2), which is why FP16 and not BF16 is the operand type.
//
// One persistent CTA per SM, 25 warps:
//   warp 0        producer: per 128x128 weight block one untiled bulk copy (TMA) of 8 KB of E2M1 codes
//                 + 1 KB of E4M3 block scales (repacked at prepare time: one contiguous 9216-byte read,
//                 each thread's 16 bytes at a conflict-free slot), and one TMA box of the FP16 B operand
//                 (32 rows x 64 k parts, 128-byte swizzle) into the same ring stage.
//   warps 9..24   dequant, four groups of four warps, group g <-> A slot g in tensor memory: thread = weight
//                 row; per 8 codes 4 cvt.rn.f16x2.e2m1x2 and 4 mul.f16x2 by the block scale (itself one
//                 cvt.rn.f16x2.e4m3x2 per two scales), written straight into tensor memory (tcgen05.st)
//                 as the A operand.  No round trip through shared memory.
//   warps 1..4    one lane each issues tcgen05.mma kind::f16, A from TMEM, B from shared memory.  One thread
//                 can issue only about one MMA per 100 clocks whatever N is, so four warps issue in parallel,
//                 each into its own FP32 accumulator in TMEM (double-buffered per unit).
//   warps 5..8    epilogue: adds the four accumulators (tcgen05.ld), times the expert's global scale (and the
//                 folded pre-expert RMSNorm row scale).  gemm 1 with one K split: gate and up rows of the same
//                 16 channels sit in the two halves of each warp (repacked so at prepare time), one shuffle
//                 brings them together and fp16(silu(gate) * up) goes straight to the B operand of gemm 2.
//                 Otherwise plain stores into this K split's FP32 partial buffer; K splits are summed in a
//                 fixed order by the consumer, so results are bitwise reproducible and no buffer has to
//                 be zeroed between calls.
// Roofline: HBM (0.5625 bytes per weight of every touched expert).
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "msk.h"
#include "ptx.cuh"
#include "route.cuh"
#include "tmap.cuh"

namespace msk {

constexpr int kBlob = 9216;        // one packed 128-row x 128-k weight block
constexpr int kBlobScales = 8192;  // offset of the 128 x 8 block scales inside a blob
constexpr int kBSlot = 8192;       // B tile of one stage: 32 rows x 256 bytes (two 128-byte-swizzled halves)
// A ring stage holds a PAIR of consecutive chunks of a unit: [weights 0][weights 1][B tile 0][B tile 1].  The
// two weight blocks are adjacent in memory and the two B tiles are one TMA box, so the single producer thread
// issues one wait, one bulk copy and one tensor copy per 2 chunks (its issue rate was the limit with one chunk
// per stage).  Units with an odd number of chunks use stages of one chunk (second halves unused).
constexpr int kStage = 2 * (kBlob + kBSlot);
#ifndef MSK_MOE_NRAW
#define MSK_MOE_NRAW 5
#endif
constexpr int kNRaw = MSK_MOE_NRAW;  // ring stages
static_assert(kNRaw >= 4, "a dequant group steps up to 4 stages at a time and wraps at most once per step");
// nanoseconds a waiting warp of each role sleeps between polls (the dequant warps, which bound the rate, poll)
constexpr int kSleepProducer = 200, kSleepIssuer = 40, kSleepEpilogue = 60;
constexpr int kNA = 4;             // A slots in tensor memory, 64 columns each
constexpr int kGroup = 32;         // pairs per expert-group (UMMA N)
constexpr int kMaxPairs = 2048;
constexpr int kMaxExperts = 256;
constexpr int kMaxGroups = 320;
constexpr int kMaxDevices = 64;     // per-device host state (function attributes, the built-in scratch's address)
constexpr int kIssuers = 4;         // MMA-issuing warps (one lane each); a single thread issues one tcgen05.mma per ~100 clk
constexpr int kDqGroups = 4;        // dequant warp groups (4 warps each); group g takes the chunks with index = g (mod 4)
static_assert(kNA == kIssuers && kNA == kDqGroups && (kIssuers & (kIssuers - 1)) == 0,
              "A slot g is written by dequant group g and read by issuing warp g: both see every phase of its barriers");
constexpr int kMoeThreads = (1 + kIssuers + 4 + 4 * kDqGroups) * 32;
constexpr int kRouteThreads = kMoeThreads, kRouteWarps = kRouteThreads / 32;

// ---------------------------------------------------------------- weight repacking (prepare time)
// Row of the [R, K] matrix that packed row r of 128-row tile rt holds.  Plain matrices: rt * 128 + r.
// gate_up matrices (inner = I > 0, rows [0, I) gate, [I, 2I) up): every 32 packed rows hold 16 gate rows followed
// by the 16 up rows of the same channels, so that one warp of the GEMM epilogue (32 accumulator lanes) owns
// both arguments of silu(gate) * up: channel = rt * 64 + (r / 32) * 16 + r % 16, up if (r / 16) is odd.
__host__ __device__ __forceinline__ int packed_src_row(int rt, int r, int inner) {
    if (inner == 0) return rt * 128 + r;
    const int ch = rt * 64 + (r >> 5) * 16 + (r & 15);
    return ((r >> 4) & 1) ? inner + ch : ch;
}

// One block = 4 quarters (32 k each) x 128 rows x 16 bytes of codes as stored (two per byte, even k in the low
// nibble), then 128 rows x 8 block scales.
__global__ void moe_pack_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ sf,
                                uint8_t* __restrict__ packed, int R, int K, int inner) {
    const int kc = blockIdx.x, rt = blockIdx.y, e = blockIdx.z, r = threadIdx.x;
    const int KC = K / 128, tiles = R / 128;
    const size_t row = static_cast<size_t>(e) * R + packed_src_row(rt, r, inner);
    uint8_t* blob = packed + ((static_cast<size_t>(e) * tiles + rt) * KC + kc) * kBlob;
    for (int q = 0; q < 4; ++q)
        *reinterpret_cast<uint4*>(blob + q * 2048 + r * 16) =
            *reinterpret_cast<const uint4*>(codes + row * (K / 2) + (kc * 128 + q * 32) / 2);
    *reinterpret_cast<uint2*>(blob + kBlobScales + r * 8) =
        *reinterpret_cast<const uint2*>(sf + row * (K / 16) + kc * 8);
}

// ---------------------------------------------------------------- dequantisation
__device__ __forceinline__ uint32_t hmul2_f16(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
// two E4M3 block scales (bits 0..15 of `two`) -> FP16x2 (s0, s1), exact (E4M3 subnormals are FP16 normals)
__device__ __forceinline__ uint32_t scale_pair(uint32_t two) {
    uint32_t d;
    asm("{\n"
        ".reg .b16 t;\n"
        "cvt.u16.u32 t, %1;\n"
        "cvt.rn.f16x2.e4m3x2 %0, t;\n"
        "}\n"
        : "=r"(d)
        : "r"(two));
    return d;
}
// 8 codes (one word: byte i holds k = 2i in its low and k = 2i + 1 in its high nibble) -> 4 FP16x2 registers
// holding value * block scale, k ascending, low half first.  s2 = the scale in both halves.
__device__ __forceinline__ void dequant_word(uint32_t w, uint32_t s2, uint32_t* r) {
    uint32_t v0, v1, v2, v3;
    asm("{\n"
        ".reg .b8 b0, b1, b2, b3;\n"
        "mov.b32 {b0, b1, b2, b3}, %4;\n"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n"
        "cvt.rn.f16x2.e2m1x2 %1, b1;\n"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n"
        "cvt.rn.f16x2.e2m1x2 %3, b3;\n"
        "}\n"
        : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3)
        : "r"(w));
    r[0] = hmul2_f16(v0, s2);
    r[1] = hmul2_f16(v1, s2);
    r[2] = hmul2_f16(v2, s2);
    r[3] = hmul2_f16(v3, s2);
}
// one thread's 32 codes (16 bytes) and their 2 block scales (FP16x2) -> 16 registers
__device__ __forceinline__ void dequant_quarter(const uint4 w, uint32_t pair, uint32_t (&r)[16]) {
    const uint32_t s0 = __byte_perm(pair, 0, 0x1010), s1 = __byte_perm(pair, 0, 0x3232);
    dequant_word(w.x, s0, r + 0);
    dequant_word(w.y, s0, r + 4);
    dequant_word(w.z, s1, r + 8);
    dequant_word(w.w, s1, r + 12);
}

// Dequantise packed blocks into plain BF16 [rows, K] in the matrix's own row order (value * block scale, no
// global scale; exact in BF16 too): test hook for the bit-exactness of the in-kernel dequantisation.
__global__ void moe_dequant_kernel(const uint8_t* __restrict__ packed, __nv_bfloat16* __restrict__ out, int R, int K,
                                   int inner) {
    const int kc = blockIdx.x, rt = blockIdx.y, e = blockIdx.z, r = threadIdx.x;
    const int KC = K / 128, tiles = R / 128;
    const uint8_t* blob = packed + ((static_cast<size_t>(e) * tiles + rt) * KC + kc) * kBlob;
    const uint2 sc = *reinterpret_cast<const uint2*>(blob + kBlobScales + r * 8);
    const uint32_t pairs[4] = {scale_pair(sc.x), scale_pair(sc.x >> 16), scale_pair(sc.y), scale_pair(sc.y >> 16)};
    __nv_bfloat16* dst = out + (static_cast<size_t>(e) * R + packed_src_row(rt, r, inner)) * K + kc * 128;
    for (int q = 0; q < 4; ++q) {
        uint32_t v[16];
        dequant_quarter(*reinterpret_cast<const uint4*>(blob + q * 2048 + r * 16), pairs[q], v);
        for (int i = 0; i < 16; ++i) {
            const __half2 h = *reinterpret_cast<const __half2*>(&v[i]);
            dst[q * 32 + 2 * i] = __float2bfloat16(__low2float(h));
            dst[q * 32 + 2 * i + 1] = __float2bfloat16(__high2float(h));
        }
    }
}

// ---------------------------------------------------------------- routing tables (rebuilt by every CTA)
struct RouteArgs {
    const int* ids;       // [T, top_k] given expert ids (ignored when logits != null)
    const float* logits;  // [T, ld_logits] router logits, or null
    int n_logits, ld_logits;
    int* ids_out;         // published by CTA 0 when routing from logits
    float* wts_out;
    int T, top_k, local_start, local_count;
    int ld_ids;           // ints (floats) between token rows of ids / wts
};

struct RouteTables {
    int n_groups, n_local;
    int counts[kMaxExperts];
    int offs[kMaxExperts + 1];
    unsigned short ids_s[kMaxPairs];   // expert id of every pair (65535 = none)
    unsigned short pos_s[kMaxPairs];   // in the end: row of every pair in `list` (65535 = not a local pair)
    unsigned short list[kMaxPairs];    // pairs sorted by (local expert, pair index)
    unsigned short g_expert[kMaxGroups], g_off[kMaxGroups], g_n[kMaxGroups];
    unsigned short seg_cnt[kRouteWarps][kMaxExperts];  // pairs per (warp segment, expert)
    int r_ids[kRouteWarps][8];
    float r_w[kRouteWarps][8];
};

// Builds the tables from ids (or logits).  Called by all kRouteThreads threads of a CTA; the result is
// the same in every CTA and every kernel (pure counting, no atomics): an expert's list is cut into
// groups that different CTAs and kernels work on, so its order must not depend on who built it.
__device__ void build_routing(RouteTables& rt, const RouteArgs& a, int* status, int where) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int P = a.T * a.top_k;
    if (a.logits != nullptr) {
        for (int t = warp; t < a.T; t += kRouteWarps) {
            route_token(a.logits + static_cast<size_t>(t) * a.ld_logits, a.n_logits, a.top_k, lane, rt.r_ids[warp], rt.r_w[warp]);
            __syncwarp();
            if (lane < a.top_k) {
                rt.ids_s[t * a.top_k + lane] = static_cast<unsigned short>(rt.r_ids[warp][lane]);
                if (blockIdx.x == 0 && a.ids_out != nullptr) {
                    a.ids_out[t * a.ld_ids + lane] = rt.r_ids[warp][lane];
                    a.wts_out[t * a.ld_ids + lane] = rt.r_w[warp][lane];
                }
            }
            __syncwarp();
        }
    } else {
        for (int i = tid; i < P; i += kRouteThreads) {
            const int id = __ldcg(a.ids + (i / a.top_k) * a.ld_ids + i % a.top_k);
            rt.ids_s[i] = static_cast<unsigned short>(id < 0 || id > 65534 ? 65535 : id);
        }
    }
    for (int i = lane; i < kMaxExperts; i += 32) rt.seg_cnt[warp][i] = 0;
    __syncthreads();
    // position of a pair in its expert's list = number of earlier pairs of that expert: each warp ranks a
    // contiguous segment (match_any inside 32-pair chunks), then the segments are prefix-summed per expert
    const int seg = ((P + kRouteWarps - 1) / kRouteWarps + 31) & ~31;
    for (int c0 = warp * seg; c0 < min(P, (warp + 1) * seg); c0 += 32) {
        const int i = c0 + lane;
        int e = i < P ? static_cast<int>(rt.ids_s[i]) - a.local_start : -1;
        if (e >= a.local_count) e = -1;
        const unsigned same = __match_any_sync(0xffffffffu, e);
        const int rank = __popc(same & ((1u << lane) - 1u));
        const int before = e >= 0 ? rt.seg_cnt[warp][e] : 0;
        __syncwarp();
        if (e >= 0) {
            rt.pos_s[i] = static_cast<unsigned short>(before + rank);
            if (rank == 0) rt.seg_cnt[warp][e] = static_cast<unsigned short>(before + __popc(same));
        }
        __syncwarp();
    }
    __syncthreads();
    for (int e = tid; e < a.local_count; e += kRouteThreads) {
        int run = 0;
        for (int w = 0; w < kRouteWarps; ++w) {
            const int c = rt.seg_cnt[w][e];
            rt.seg_cnt[w][e] = static_cast<unsigned short>(run);
            run += c;
        }
        rt.counts[e] = run;
    }
    __syncthreads();
    if (warp == 0) {
        // offsets and expert-groups by a warp scan: lane l owns experts 8 l .. 8 l + 7.  (One thread walking all
        // the experts costs ~200 clocks per expert: dependent single-thread issue.)
        int n_[8], sum_n = 0, sum_g = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = lane * 8 + i;
            n_[i] = e < a.local_count ? rt.counts[e] : 0;
            sum_n += n_[i];
            sum_g += (n_[i] + kGroup - 1) / kGroup;
        }
        int inc_n = sum_n, inc_g = sum_g;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int vn = __shfl_up_sync(0xffffffffu, inc_n, o), vg = __shfl_up_sync(0xffffffffu, inc_g, o);
            if (lane >= o) inc_n += vn, inc_g += vg;
        }
        int off = inc_n - sum_n, gi = inc_g - sum_g;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = lane * 8 + i;
            if (e < a.local_count) {
                rt.offs[e] = off;
                for (int g = 0; g < n_[i]; g += kGroup, ++gi) {
                    if (gi < kMaxGroups) {
                        rt.g_expert[gi] = static_cast<unsigned short>(e);
                        rt.g_off[gi] = static_cast<unsigned short>(off + g);
                        rt.g_n[gi] = static_cast<unsigned short>(min(kGroup, n_[i] - g));
                    } else {
                        report(status, MSK_ERR_CAPACITY, where | 1, gi, kMaxGroups);
                    }
                }
                off += n_[i];
            }
        }
        if (lane == 31) {
            rt.n_groups = min(inc_g, kMaxGroups);
            rt.n_local = inc_n;
        }
    }
    __syncthreads();
    for (int i = tid; i < P; i += kRouteThreads) {
        const int e = static_cast<int>(rt.ids_s[i]) - a.local_start;
        if (e >= 0 && e < a.local_count) {
            const int dst = rt.offs[e] + rt.seg_cnt[i / seg][e] + rt.pos_s[i];
            rt.list[dst] = static_cast<unsigned short>(i);
            rt.pos_s[i] = static_cast<unsigned short>(dst);
        } else {
            rt.pos_s[i] = 65535;
        }
    }
    __syncthreads();
}

// Up to 32 tokens: the same tables from one warp, in a fraction of the code (this runs at the head of every GEMM
// CTA, from a cold instruction cache, before the first weight byte can be requested).  A token meets an expert at
// most once, so an expert's pairs are a 32-bit token mask and every touched expert is exactly one group:
//   g_expert / g_off / g_n as above, offs[g] = token mask of group g, ids_s = the ids.  Row r of an expert's list
//   is its r-th token in ascending order: the same order build_routing produces.
// list / pos_s are not filled: only gemm 1 in its token-per-column form uses these tables, and there a pair's row
// follows from its expert's mask (see the epilogue).
__device__ void build_routing_small(RouteTables& rt, const RouteArgs& a, int lane) {
    const int P = a.T * a.top_k;
    unsigned* emask = reinterpret_cast<unsigned*>(rt.counts);  // per local expert: tokens routed to it
    for (int e = lane; e < kMaxExperts; e += 32) emask[e] = 0u;
    __syncwarp();
    for (int i = lane; i < P; i += 32) {
        const int id = __ldcg(a.ids + (i / a.top_k) * a.ld_ids + i % a.top_k);
        rt.ids_s[i] = static_cast<unsigned short>(id < 0 || id > 65534 ? 65535 : id);
        const int e = id - a.local_start;
        if (e >= 0 && e < a.local_count) atomicOr(&emask[e], 1u << (i / a.top_k));
    }
    __syncwarp();
    // lane l owns experts 8 l .. 8 l + 7: exclusive scans of (touched, pairs) over the warp
    unsigned m[8];
    int touched = 0, pairs = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int e = lane * 8 + i;
        m[i] = e < a.local_count ? emask[e] : 0u;
        touched += m[i] != 0u;
        pairs += __popc(m[i]);
    }
    int inc_t = touched, inc_p = pairs;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int vt = __shfl_up_sync(0xffffffffu, inc_t, o), vp = __shfl_up_sync(0xffffffffu, inc_p, o);
        if (lane >= o) inc_t += vt, inc_p += vp;
    }
    int gi = inc_t - touched, off = inc_p - pairs;
    __syncwarp();  // emask (aliasing counts) has been read by everyone
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (m[i] == 0u) continue;
        rt.g_expert[gi] = static_cast<unsigned short>(lane * 8 + i);
        rt.g_off[gi] = static_cast<unsigned short>(off);
        rt.g_n[gi] = static_cast<unsigned short>(__popc(m[i]));
        rt.offs[gi] = static_cast<int>(m[i]);
        off += __popc(m[i]);
        ++gi;
    }
    if (lane == 31) rt.n_groups = inc_t, rt.n_local = inc_p;
}

// ---------------------------------------------------------------- B-operand helpers
// FP16 copy of the expert input.  Up to 32 tokens: row = token (the GEMM's B tile is the tokens themselves).
// More: rows in expert-list order, so that an expert-group's B tile is one TMA box.
struct MoeStageArgs {
    RouteArgs route;
    const void* x;     // [T, ldx] BF16, or FP16 when x_fp16
    int ldx, H, x_fp16, direct;
    __half* x16;       // [T, H] (direct) or [T*top_k, H]
    const int* wait_flags;  // expert parallelism: the rows of x arrive from other GPUs; entry i >= wait_value when
    int wait_count, wait_value;  // source i's rows are complete
    long long wait_cycles;
    int* status;
};

__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t v) {
    const float lo = fminf(fmaxf(bf16lo(v), -65504.0f), 65504.0f), hi = fminf(fmaxf(bf16hi(v), -65504.0f), 65504.0f);
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

__global__ void __launch_bounds__(kRouteThreads) moe_stage_kernel(MoeStageArgs p) {
    __shared__ RouteTables rt;
    pdl_wait();
    pdl_launch_dependents();
    if (p.wait_flags != nullptr) {
        if (static_cast<int>(threadIdx.x) < p.wait_count)
            flag_wait_ge(p.wait_flags + threadIdx.x, p.wait_value, p.wait_cycles, p.status, (MSK_K_EP << 8) | 1);
        __syncthreads();
    }
    int n_rows = p.route.T;
    if (!p.direct) {
        RouteArgs ra = p.route;
        ra.ids_out = nullptr;
        build_routing(rt, ra, p.status, MSK_K_MOE1 << 8);
        n_rows = rt.n_local;
    }
    const int tid = threadIdx.x;
    for (int r = blockIdx.x; r < n_rows; r += gridDim.x) {
        const int tok = p.direct ? r : rt.list[r] / p.route.top_k;
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.x) + static_cast<size_t>(tok) * p.ldx);
        uint4* dst = reinterpret_cast<uint4*>(p.x16 + static_cast<size_t>(r) * p.H);
        for (int i = tid; i < p.H / 8; i += kRouteThreads) {
            uint4 v = __ldcg(src + i);
            if (!p.x_fp16) v = make_uint4(bf16x2_to_f16x2(v.x), bf16x2_to_f16x2(v.y), bf16x2_to_f16x2(v.z), bf16x2_to_f16x2(v.w));
            dst[i] = v;
        }
    }
}

__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.0f + __expf(-g)) * u; }
__device__ __forceinline__ float clamp_f16(float v) { return fminf(fmaxf(v, -65504.0f), 65504.0f); }

// Activation between the two GEMMs when gemm 1 ran with K splits (its epilogue then cannot apply it):
// inter[r] = fp16(silu(gate) * up) of the r-th pair in expert-list order.  The partial rows are in packed row
// order (see packed_src_row): channel j sits at column (j / 64) * 128 + (j % 64 / 16) * 32 + j % 16, its up
// value 16 columns further.
struct MoeActArgs {
    const int* route_pub;  // [0] = local pairs, [2 + r] = pair of sorted row r (published by gemm 1)
    const float* h1;       // [s1][P][2I]
    int s1, P, inner;
    __half* inter;         // [P, I]
};

__global__ void __launch_bounds__(256) moe_act_kernel(MoeActArgs p) {
    pdl_wait();
    pdl_launch_dependents();
    const int n_local = __ldcg(p.route_pub);
    for (int r = blockIdx.x; r < n_local; r += gridDim.x) {
        const int pair = __ldcg(p.route_pub + 2 + r);
        for (int k = threadIdx.x * 4; k < p.inner; k += 1024) {
            const int col = (k >> 6) * 128 + ((k >> 4) & 3) * 32 + (k & 15);
            float4 g = make_float4(0, 0, 0, 0), u = make_float4(0, 0, 0, 0);
            for (int s = 0; s < p.s1; ++s) {
                const float* row = p.h1 + (static_cast<size_t>(s) * p.P + pair) * (2 * p.inner) + col;
                const float4 a = __ldcg(reinterpret_cast<const float4*>(row));
                const float4 c = __ldcg(reinterpret_cast<const float4*>(row + 16));
                g.x += a.x, g.y += a.y, g.z += a.z, g.w += a.w;
                u.x += c.x, u.y += c.y, u.z += c.z, u.w += c.w;
            }
            const __half2 o01 = __floats2half2_rn(clamp_f16(silu_mul(g.x, u.x)), clamp_f16(silu_mul(g.y, u.y)));
            const __half2 o23 = __floats2half2_rn(clamp_f16(silu_mul(g.z, u.z)), clamp_f16(silu_mul(g.w, u.w)));
            *reinterpret_cast<uint2*>(p.inter + static_cast<size_t>(r) * p.inner + k) =
                make_uint2(*reinterpret_cast<const uint32_t*>(&o01), *reinterpret_cast<const uint32_t*>(&o23));
        }
    }
}

// ---------------------------------------------------------------- grouped GEMM
struct MoeGemmArgs {
    RouteArgs route;
    const uint8_t* wpacked;
    const float* gs;   // [local_count]
    int R, K;          // rows and reduction length per expert
    int direct;        // gemm 1 with <= 32 tokens: B rows are the tokens themselves (column = token)
    const float* x_ssq;
    int x_ssq_parts, x_ssq_ts;
    float x_inv_dim, x_eps;
    int* route_pub;    // gemm 1, CTA 0: [0] local pairs, [1] groups, [2 + r] pair of sorted row r
    float* outp;       // [S][T*top_k][R] FP32 partials (not written when fuse_act)
    __half* inter;     // gemm 1, fuse_act: [T*top_k, inner] activations, rows in expert-list order
    int inner, fuse_act;
    int S;
    int route_early;   // the routing input is final before the previous kernel ends
    int small;         // <= 32 tokens, ids given: one warp builds the compact tables (build_routing_small)
    int share_chunks;  // 1: the issuing warps split every chunk's K steps (short units); 0: a warp per A slot
    int* status;
};

struct MoeBars {
    // raw_full: two barriers per ring stage, used by the stage's even and odd fills.  A dequant group does not see
    // every fill of a stage (its sibling groups take the chunks in between), so with one barrier per stage its
    // parity wait could meet a barrier still one fill behind - when a later stage's copies land before an earlier
    // one's - and pass on the parity of two fills ago.  With alternating barriers a barrier's previous fill is two
    // fills of the stage back, and that one was consumed before the stage could be refilled at all.
    uint64_t raw_full[2][kNRaw], raw_empty[kNRaw], a_full[kNA], a_empty[kNA], d_full[2], d_empty[2];
    uint32_t tmem_slot;
};

template <int MODE>
__global__ void __launch_bounds__(kMoeThreads, 1) moe_gemm_kernel(const __grid_constant__ CUtensorMap tm_b, MoeGemmArgs p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) MoeBars bar;
    __shared__ RouteTables rt;
    __shared__ float rs_s[kMaxPairs / 8];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int where = (MODE == 1 ? MSK_K_MOE1 : MSK_K_MOE2) << 8;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
    const int P = p.route.T * p.route.top_k;

    if (warp == 0) {
        tmem_alloc(smem_u32(&bar.tmem_slot), 512);
        tmem_relinquish();
    }
    const int psh = ((p.K / 128 / p.S) & 1) ? 0 : 1;  // log2(chunks per ring stage)
    if (tid == 32) {
        // a ring stage (weight block + B tile) is free again when the 4 dequant warps have read the block and
        // the MMAs that read the B tile (one issuing warp per chunk) have completed
        for (int i = 0; i < kNRaw; ++i) {
            mbar_init(smem_u32(&bar.raw_full[0][i]), 1), mbar_init(smem_u32(&bar.raw_full[1][i]), 1);
            mbar_init(smem_u32(&bar.raw_empty[i]), (4 + (p.share_chunks ? kIssuers : 1)) << psh);
        }
        for (int i = 0; i < kNA; ++i) mbar_init(smem_u32(&bar.a_full[i]), 4), mbar_init(smem_u32(&bar.a_empty[i]), p.share_chunks ? kIssuers : 1);
        for (int i = 0; i < 2; ++i) mbar_init(smem_u32(&bar.d_full[i]), kIssuers), mbar_init(smem_u32(&bar.d_empty[i]), 4);
        fence_mbar_init();
    }
    if (tid == 0) prefetch_tmap(&tm_b);
    // The expert ids are complete before this kernel can start whenever its predecessor in the stream is one
    // of this file's own kernels (gather, activation): those release their dependents only after their own
    // wait on the kernel before them.  The tables are then built while the predecessor still runs.
    auto route = [&]() {
        if (p.small) {
            if (warp == 0) build_routing_small(rt, p.route, lane);
            __syncthreads();
        } else {
            build_routing(rt, p.route, p.status, where);
        }
    };
    if (p.route_early) route();
    pdl_wait();  // x and the gemm-1 activations come from the previous kernels
    pdl_launch_dependents();
    if (!p.route_early) route();
    if (MODE == 1 && p.x_ssq != nullptr) {
        for (int t = tid; t < p.route.T; t += kMoeThreads) {
            float s = 0.0f;
            for (int part = 0; part < p.x_ssq_parts; ++part)
                s += __ldcg(p.x_ssq + (static_cast<size_t>(part) * p.route.T + t) * p.x_ssq_ts);
            rs_s[t] = rsqrtf(s * p.x_inv_dim + p.x_eps);
        }
    }
    if (MODE == 1 && blockIdx.x == 0 && p.route_pub != nullptr && !p.small) {
        if (tid == 0) p.route_pub[0] = rt.n_local, p.route_pub[1] = rt.n_groups;
        for (int r = tid; r < rt.n_local; r += kMoeThreads) p.route_pub[2 + r] = rt.list[r];
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bar.tmem_slot;

    const int tiles = p.R / 128, KC = p.K / 128, nch = KC / p.S;
    const int per_group = tiles * p.S;
    const int n_units = rt.n_groups * per_group;

    if (warp == 0) {
        // ------------------------------------------------ producer: weight block (bulk copy) + B tile (2 TMA boxes)
        if (lane == 0) {
            int pc = 0, s = 0, sph = 1, fill = 0;  // stages filled so far, stage, parity of the stage's previous use, fills of the stage so far
            const int per = 1 << psh;
            bool ok = true;
            for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
                const int g = u / per_group, rem = u % per_group, tile = rem / p.S, ks = rem % p.S;
                const uint8_t* src = p.wpacked + ((static_cast<size_t>(rt.g_expert[g]) * tiles + tile) * KC + ks * nch) * kBlob;
                const int row0 = p.direct ? 0 : rt.g_off[g];
                const int kg0 = ks * nch * 2;  // 64-column group of the B operand
                // every CTA reads the same B tiles (direct mode) for the same k: unit u starts its K range at a
                // different stage, so that the CTAs do not pull the same lines from the same L2 slices together
                const int nstg = nch >> psh;
                int ii = u % nstg;
                for (int c = 0; c < nch; c += per, ++pc) {
                    if (pc >= kNRaw) ok = mbar_wait<kSleepProducer>(smem_u32(&bar.raw_empty[s]), sph, p.status, where | 2);
                    if (!ok) break;
                    const uint32_t full = smem_u32(&bar.raw_full[fill & 1][s]), dst = base + s * kStage;
                    mbar_expect_tx(full, per * kBlob + 2 * kBSlot);  // the B box always spans 2 chunks
                    bulk_load(dst, src + static_cast<size_t>(ii) * (per * kBlob), per * kBlob, full);
                    tma_load_3d(dst + 2 * kBlob, &tm_b, full, 0, row0, kg0 + ii * 2 * per);
                    if (++ii == nstg) ii = 0;
                    if (++s == kNRaw) s = 0, sph ^= 1, ++fill;
                }
            }
        }
        __syncwarp();
    } else if (warp <= kIssuers) {
        // ------------------------------------------------ MMA issue.  One thread issues an MMA per ~110 cycles, so
        // four threads share the work, each into its own accumulator; the epilogue adds the accumulators.
        //   long units:  issuing warp w owns A slot w, i.e. every chunk with (running chunk number) % 4 == w, and
        //                issues its 8 K steps.  Owning a slot, a warp sees every phase of that slot's barrier in
        //                order (a parity wait must never skip a phase).
        //   short units (few tokens, many K splits): every warp issues 2 of the 8 K steps of every chunk, so a
        //                chunk is through after 2 issue times instead of 8.
        // a_full implies raw_full: the dequant warps waited for the stage before they wrote the A slot.
        // This thread shares its scheduler with five busy warps, so every instruction of its sequential loop costs
        // tens of cycles: it visits only its own chunks and steps stage, slot and phases instead of dividing.
        if (lane == 0) {
            const int w = warp - 1;
            const uint32_t idesc = umma_idesc(128, kGroup, 0, 0, 0, 0);  // FP16 x FP16 -> FP32
            const int step = p.share_chunks ? 1 : kIssuers;         // chunks between two of this warp's chunks
            const int sstep = p.share_chunks ? 0 : (kIssuers >> psh);  // ring stages between them (share: see below)
            int c = p.share_chunks ? 0 : w, cc = c;                  // place in the unit, running chunk number
            int s = (cc >> psh) % kNRaw, as = cc % kNA, aph = 0, uc = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x, ++uc) {
                const int db = uc & 1;
                if (uc >= 2) ok = mbar_wait<kSleepIssuer>(smem_u32(&bar.d_empty[db]), ((uc >> 1) - 1) & 1, p.status, where | 3);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d = tmem + kNA * 64 + (db * kIssuers + w) * kGroup;
                bool first = true;
                for (; c < nch; c += step, cc += step) {
                    ok = mbar_wait<kSleepIssuer>(smem_u32(&bar.a_full[as]), aph, p.status, where | 4);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a0 = tmem + as * 64;
                    const uint64_t b0 = umma_smem_desc(base + s * kStage + 2 * kBlob + (cc & ((1 << psh) - 1)) * kBSlot, 16, 1024, kSwizzle128);
                    if (p.share_chunks) {  // K steps 2w and 2w + 1
                        const uint64_t bd = b0 + (w >> 1) * 256 + 4 * (w & 1);
                        umma_f16_ts(d, a0 + 16 * w, bd, idesc, !first);
                        umma_f16_ts(d, a0 + 16 * w + 8, bd + 2, idesc, 1);
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j)  // K step j: 8 columns of A, 32 bytes of a B row, second half 4096 B on
                            umma_f16_ts(d, a0 + 8 * j, b0 + (j < 4 ? 0 : 256) + 2 * (j & 3), idesc, !first || j != 0);
                    }
                    first = false;
                    umma_commit(smem_u32(&bar.a_empty[as]));
                    umma_commit(smem_u32(&bar.raw_empty[s]));
                    if (p.share_chunks) {  // every chunk: next slot, next stage every 2^psh chunks
                        if (++as == kNA) as = 0, aph ^= 1;
                        if (((cc + 1) & ((1 << psh) - 1)) == 0 && ++s == kNRaw) s = 0;
                    } else {               // own slot; its barrier flips every visit
                        aph ^= 1;
                        s += sstep;
                        if (s >= kNRaw) s -= kNRaw;
                    }
                }
                c -= nch;
                if (ok) umma_commit(smem_u32(&bar.d_full[db]));
            }
        }
        __syncwarp();
    } else if (warp < kIssuers + 5) {
        // ------------------------------------------------ epilogue
        const int quarter = warp & 3, row = quarter * 32 + lane;
        int uc = 0, cc0 = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x, ++uc, cc0 += nch) {
            const int g = u / per_group, rem = u % per_group, tile = rem / p.S, ks = rem % p.S;
            const int db = uc & 1, e = rt.g_expert[g], off = rt.g_off[g], n = rt.g_n[g];
            // the pair whose result sits in accumulator column `lane`
            int mypair = -1, myrow = -1;  // myrow: the pair's place in the expert-ordered list (row of `inter`)
            if (p.direct) {  // column = token
                if (lane < p.route.T)
                    for (int sl = 0; sl < p.route.top_k; ++sl)
                        if (static_cast<int>(rt.ids_s[lane * p.route.top_k + sl]) == e + p.route.local_start) mypair = lane * p.route.top_k + sl;
                // compact tables: the row follows from the expert's token mask
                if (mypair >= 0) myrow = p.small ? off + __popc(static_cast<unsigned>(rt.offs[g]) & ((1u << lane) - 1u)) : rt.pos_s[mypair];
            } else if (lane < n) {
                mypair = rt.list[off + lane];
                myrow = off + lane;
            }
            const float myscale = (MODE == 1 && p.x_ssq != nullptr && mypair >= 0) ? rs_s[mypair / p.route.top_k] : 1.0f;
            // gemm 1 applies the expert's global scale (requested before the wait); gemm 2 leaves it, like everything
            // else that is per expert or per pair, to the combine kernel: its epilogue bounds the rate at many tokens
            const float scale = MODE == 1 ? __ldg(p.gs + e) : 1.0f;
            const int myoff = mypair >= 0 ? mypair * p.R : -1;  // of the pair's row in a partial plane
            ok = mbar_wait<kSleepEpilogue>(smem_u32(&bar.d_full[db]), (uc >> 1) & 1, p.status, where | 6);
            if (!ok) break;
            tc_fence_after();
            float* dst = p.outp + (static_cast<size_t>(ks) * P) * p.R + tile * 128 + row;
            // channel of this lane's gate row (lanes 0..15 of a warp hold gate rows, 16..31 the up rows of the same channels)
            __half* dst_act = p.inter + tile * 64 + quarter * 16 + (lane & 15);
            // Eight accumulator columns per step, only the columns in use, in a rolled loop: this code runs once per
            // unit and unrolled it was mostly instruction fetch (with short units, gemm 2, the epilogue bounded the
            // rate).  The accumulators of issuing warps that had no chunk in this unit hold stale values: skipped.
            const uint32_t taddr = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + kNA * 64 + db * kIssuers * kGroup;
            unsigned has = 0;
#pragma unroll
            for (int w = 0; w < kIssuers; ++w)
                if (p.share_chunks || ((w - cc0) & (kIssuers - 1)) < nch) has |= 1u << w;
            // columns that hold a pair of this expert (in direct mode most tokens have none)
            const unsigned cols = __ballot_sync(0xffffffffu, mypair >= 0);
            const int last8 = cols ? (31 - __clz(cols)) & ~7 : 0;  // the last group of 8 columns with work
#pragma unroll 1
            for (int c0 = 0; c0 <= last8; c0 += 8) {
                if (((cols >> c0) & 0xFFu) == 0) continue;
                uint32_t t[kIssuers][8];
#pragma unroll
                for (int w = 0; w < kIssuers; ++w)
                    if (has & (1u << w)) tmem_ld8(taddr + w * kGroup + c0, t[w]);
                tmem_wait_ld();
                if (c0 == last8) {  // last read of this accumulator buffer
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bar.d_empty[db]));
                }
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    float v = 0.0f;
#pragma unroll
                    for (int w = 0; w < kIssuers; ++w)
                        if (has & (1u << w)) v += __uint_as_float(t[w][c]);
                    if (MODE == 1) v *= scale * __shfl_sync(0xffffffffu, myscale, c0 + c);
                    if (MODE == 1 && p.fuse_act) {
                        const int sr = __shfl_sync(0xffffffffu, myrow, c0 + c);
                        const float up = __shfl_xor_sync(0xffffffffu, v, 16);
                        if (sr >= 0 && lane < 16) dst_act[static_cast<size_t>(sr) * p.inner] = __float2half_rn(clamp_f16(silu_mul(v, up)));
                    } else {
                        const int off = __shfl_sync(0xffffffffu, myoff, c0 + c);
                        if (off >= 0) dst[off] = v;
                    }
                }
            }
            if (cols == 0) {  // never the case for a unit that exists; keeps the barrier protocol whole
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bar.d_empty[db]));
            }
        }
    } else {
        // ------------------------------------------------ dequant: codes + scales -> BF16 A operand in TMEM
        // (all 8 warps on the same chunk was measured slower: the per-chunk handshakes then cost every warp)
        const int quarter = warp & 3, grp = (warp - (kIssuers + 5)) >> 2, row = quarter * 32 + lane;
        // the dequant warps do not care about unit boundaries: group g takes chunks g, g + 2, ... of this CTA's
        // stream; stage, slot and their phases are stepped, not divided
        const int my_units = blockIdx.x < n_units ? (n_units - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
        const int total = my_units * nch;
        bool ok = true;
        int s = (grp >> psh) % kNRaw, fill = 0, aph = 0;  // ring stage of the group's chunk, fills of that stage before it
        const int as = grp;  // this group's A slot
        const int sub = grp & ((1 << psh) - 1), sstep = kDqGroups >> psh;  // place in the stage; stages per step
        for (int cc = grp; cc < total && ok; cc += kDqGroups) {
            {
                ok = mbar_wait(smem_u32(&bar.raw_full[fill & 1][s]), (fill >> 1) & 1, p.status, where | 7);
                if (ok && cc >= kNA) ok = mbar_wait(smem_u32(&bar.a_empty[as]), aph ^ 1, p.status, where | 8);
                if (!ok) break;
                tc_fence_after();
                const uint8_t* raw = gbase + s * kStage + sub * kBlob;
                const uint2 sc = *reinterpret_cast<const uint2*>(raw + kBlobScales + row * 8);
                const uint32_t pairs[4] = {scale_pair(sc.x), scale_pair(sc.x >> 16), scale_pair(sc.y), scale_pair(sc.y >> 16)};
                const uint32_t taddr = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + as * 64;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint32_t r[16];
                    dequant_quarter(*reinterpret_cast<const uint4*>(raw + q * 2048 + row * 16), pairs[q], r);
                    tmem_st16(taddr + q * 16, r);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bar.raw_empty[s]));
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bar.a_full[as]));
                s += sstep;
                if (s >= kNRaw) s -= kNRaw, ++fill;  // sstep <= 4 <= kNRaw: at most one wrap
                aph ^= 1;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------- post-expert norm + weighted combine
struct MoeCombineArgs {
    const int* ids;
    const float* wts;
    int top_k, local_start, local_count, H, S, P, ld_ids;
    const float* yp;            // [S][P][H]: gemm 2's sums without the experts' global scales
    const float* gs;            // [local_count] global scales of the down projections
    const __nv_bfloat16* post_w;
    float eps;
    const float* resid;
    int ldr;
    void* out;
    int out_fp32, ldo;
    __nv_bfloat16* out_copy;  // optional BF16 copy of the result
    int ldc;
    // expert parallelism: the row of token t goes to GPU t / rows_per_peer, at byte offset out_off of its region,
    // row t % rows_per_peer; tokens without a local expert send nothing.  The last block to finish sets the
    // int32 at flag_off of every peer's region to flag_value.
    void* const* peers;
    int n_peers, rows_per_peer;
    size_t out_off, flag_off;
    int flag_value;
    int* done_counter;
};

// One CTA per token, 512 threads, each owning 4 output channels per 2048 of H: all the token's slots and K
// splits are loaded back to back (memory-level parallelism instead of a dependent loop), kept in registers
// for the second pass.
constexpr int kCombineThreads = 512;

// Expert parallelism: every block, after its row is on its way, takes a ticket; the last one tells every peer
// that this GPU's partial rows of the step are complete.
__device__ __forceinline__ void combine_signal(const MoeCombineArgs& p, int tid) {
    __syncthreads();  // the block's stores, then one system-scope fence by the thread that takes the ticket
    if (tid == 0) {
        __threadfence_system();
        const int old = atomicAdd(p.done_counter, 1);
        if (old == static_cast<int>(gridDim.x) - 1) {
            *p.done_counter = 0;
            __threadfence_system();
            for (int r = 0; r < p.n_peers; ++r)
                st_relaxed_sys(reinterpret_cast<int*>(static_cast<char*>(p.peers[r]) + p.flag_off), p.flag_value);
        }
    }
}

template <int ITERS, int KS>  // ITERS * 2048 >= H; KS = K splits of gemm 2 (0: any, rolled loop)
__global__ void __launch_bounds__(kCombineThreads) moe_combine_kernel(MoeCombineArgs p) {
    __shared__ float red[kCombineThreads / 32][8];
    __shared__ float rnorm[8];
    const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_wait();
    pdl_launch_dependents();
    float* peer_row = nullptr;
    if (p.peers != nullptr)
        peer_row = reinterpret_cast<float*>(static_cast<char*>(p.peers[t / p.rows_per_peer]) + p.out_off) +
                   static_cast<size_t>(t % p.rows_per_peer) * p.ldo;
    int local[8];
    float w[8], g[8];
#pragma unroll
    for (int s = 0; s < 8; ++s) {
        local[s] = 0, w[s] = 0.0f, g[s] = 0.0f;
        if (s < p.top_k) {
            const int e = __ldcg(p.ids + t * p.ld_ids + s) - p.local_start;
            local[s] = e >= 0 && e < p.local_count;
            w[s] = __ldcg(p.wts + t * p.ld_ids + s);
            if (local[s]) g[s] = __ldg(p.gs + e);
        }
    }
    bool any_local = false;
#pragma unroll
    for (int s = 0; s < 8; ++s) any_local = any_local || local[s];
    if (p.peers != nullptr && !any_local) {  // nothing to send for this token
        combine_signal(p, tid);
        return;
    }
    float4 z[ITERS][8];
    float ss[8];
#pragma unroll
    for (int s = 0; s < 8; ++s) ss[s] = 0.0f;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int d = (tid + it * kCombineThreads) * 4;
#pragma unroll
        for (int s = 0; s < 8; ++s) z[it][s] = make_float4(0, 0, 0, 0);
        if (d >= p.H) continue;
        // every (slot, split) load is issued before any is used; a slot of another rank reads slot 0's row
        // (valid memory) and is discarded
        if constexpr (KS > 0) {
            float4 ld[8][KS];
#pragma unroll
            for (int s = 0; s < 8; ++s)
#pragma unroll
                for (int k = 0; k < KS; ++k)
                    ld[s][k] = __ldcg(reinterpret_cast<const float4*>(
                        p.yp + (static_cast<size_t>(k) * p.P + t * p.top_k + (local[s] ? s : 0)) * p.H + d));
#pragma unroll
            for (int s = 0; s < 8; ++s)
#pragma unroll
                for (int k = 0; k < KS; ++k)
                    if (local[s]) z[it][s].x += ld[s][k].x, z[it][s].y += ld[s][k].y, z[it][s].z += ld[s][k].z, z[it][s].w += ld[s][k].w;
        } else {
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                if (!local[s]) continue;
                for (int k = 0; k < p.S; ++k) {
                    const float4 a = __ldcg(reinterpret_cast<const float4*>(p.yp + (static_cast<size_t>(k) * p.P + t * p.top_k + s) * p.H + d));
                    z[it][s].x += a.x, z[it][s].y += a.y, z[it][s].z += a.z, z[it][s].w += a.w;
                }
            }
        }
        const uint2 pw = *reinterpret_cast<const uint2*>(p.post_w + d);
        const float f[4] = {1.0f + bf16lo(pw.x), 1.0f + bf16hi(pw.x), 1.0f + bf16lo(pw.y), 1.0f + bf16hi(pw.y)};
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            float4& y = z[it][s];
            y.x *= f[0] * g[s], y.y *= f[1] * g[s], y.z *= f[2] * g[s], y.w *= f[3] * g[s];
            ss[s] += y.x * y.x + y.y * y.y + y.z * y.z + y.w * y.w;
        }
    }
#pragma unroll
    for (int s = 0; s < 8; ++s) {
        const float v = warp_sum(ss[s]);
        if (lane == 0) red[warp][s] = v;
    }
    __syncthreads();
    if (tid < 8) {
        float v = 0.0f;
        for (int k = 0; k < kCombineThreads / 32; ++k) v += red[k][tid];
        rnorm[tid] = rsqrtf(v / p.H + p.eps);
    }
    __syncthreads();
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int d = (tid + it * kCombineThreads) * 4;
        if (d >= p.H) continue;
        float4 acc = make_float4(0, 0, 0, 0);
        if (p.resid != nullptr) acc = __ldcg(reinterpret_cast<const float4*>(p.resid + static_cast<size_t>(t) * p.ldr + d));
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            if (!local[s]) continue;
            const float c = w[s] * rnorm[s];
            acc.x += z[it][s].x * c, acc.y += z[it][s].y * c, acc.z += z[it][s].z * c, acc.w += z[it][s].w * c;
        }
        if (peer_row != nullptr) {
            *reinterpret_cast<float4*>(peer_row + d) = acc;
        } else if (p.out_fp32) {
            *reinterpret_cast<float4*>(static_cast<float*>(p.out) + static_cast<size_t>(t) * p.ldo + d) = acc;
        } else {
            *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(t) * p.ldo + d) =
                make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
        }
        if (p.out_copy != nullptr)
            *reinterpret_cast<uint2*>(p.out_copy + static_cast<size_t>(t) * p.ldc + d) =
                make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
    }
    if (p.peers != nullptr) combine_signal(p, tid);
}

template <typename Kern, typename Args>
static int launch_pdl(Kern kern, dim3 grid, dim3 block, int smem, cudaStream_t stream, int pdl, const Args& args) {
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
    return cudaLaunchKernelEx(&cfg, kern, args) == cudaSuccess ? 0 : MSK_ERR_CUDA;
}

template <typename Kern, typename Args>
static int launch_pdl2(Kern kern, dim3 grid, dim3 block, int smem, cudaStream_t stream, int pdl, const CUtensorMap& tm,
                       const Args& args) {
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
    return cudaLaunchKernelEx(&cfg, kern, tm, args) == cudaSuccess ? 0 : MSK_ERR_CUDA;
}

}  // namespace msk

extern "C" int msk_moe_packed_bytes(int E, int H, int I, size_t* w13_bytes, size_t* w2_bytes) {
    if (E < 1 || H % 128 != 0 || I % 128 != 0 || (2 * I) % 128 != 0) return MSK_ERR_UNSUPPORTED;
    if (w13_bytes) *w13_bytes = static_cast<size_t>(E) * (2 * I / 128) * (H / 128) * msk::kBlob;
    if (w2_bytes) *w2_bytes = static_cast<size_t>(E) * (H / 128) * (I / 128) * msk::kBlob;
    return 0;
}

extern "C" int msk_moe_pack(const MskMoeWeights* w, void* w13_packed, void* w2_packed, void* stream) {
    using namespace msk;
    if (w == nullptr || !w->w13 || !w->w13_sf || !w->w2 || !w->w2_sf || !w13_packed || !w2_packed) return MSK_ERR_INVALID;
    if (w->H % 128 != 0 || w->I % 128 != 0) return MSK_ERR_UNSUPPORTED;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    moe_pack_kernel<<<dim3(w->H / 128, 2 * w->I / 128, w->E), 128, 0, s>>>(
        static_cast<const uint8_t*>(w->w13), static_cast<const uint8_t*>(w->w13_sf), static_cast<uint8_t*>(w13_packed),
        2 * w->I, w->H, w->I);
    moe_pack_kernel<<<dim3(w->I / 128, w->H / 128, w->E), 128, 0, s>>>(
        static_cast<const uint8_t*>(w->w2), static_cast<const uint8_t*>(w->w2_sf), static_cast<uint8_t*>(w2_packed), w->H,
        w->I, 0);
    return cudaGetLastError() == cudaSuccess ? 0 : MSK_ERR_CUDA;
}

extern "C" int msk_moe_dequant(const void* packed, void* out_bf16, int E, int R, int K, int gate_up, void* stream) {
    using namespace msk;
    if (!packed || !out_bf16 || R % 128 != 0 || K % 128 != 0) return MSK_ERR_INVALID;
    moe_dequant_kernel<<<dim3(K / 128, R / 128, E), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(packed), static_cast<__nv_bfloat16*>(out_bf16), R, K, gate_up ? R / 2 : 0);
    return cudaGetLastError() == cudaSuccess ? 0 : MSK_ERR_CUDA;
}

extern "C" int msk_moe_scratch_bytes(int T, int top_k, int H, int I, int s1, int s2, size_t* h1_bytes, size_t* y_bytes,
                                     size_t* inter_bytes, size_t* x_sorted_bytes, size_t* route_bytes) {
    if (T < 1 || top_k < 1 || s1 < 1 || s2 < 1) return MSK_ERR_INVALID;
    const size_t P = static_cast<size_t>(T) * top_k;
    if (h1_bytes) *h1_bytes = s1 * P * 2 * I * sizeof(float);
    if (y_bytes) *y_bytes = s2 * P * H * sizeof(float);
    if (inter_bytes) *inter_bytes = P * I * 2;
    if (x_sorted_bytes) *x_sorted_bytes = (T > msk::kGroup ? P : static_cast<size_t>(T)) * H * 2;
    if (route_bytes) *route_bytes = (2 + P) * sizeof(int);
    return 0;
}

extern "C" int msk_moe_forward(const MskMoeParams* q, int* status, void* stream) {
    using namespace msk;
    if (q == nullptr || !q->x || !q->w13_packed || !q->w2_packed || !q->w13_gs || !q->w2_gs || !q->post_norm_w ||
        !q->y_part || !q->inter_sorted || !q->topk_ids || !q->topk_weights)
        return MSK_ERR_INVALID;
    if (!q->out && !(q->ep != nullptr && q->ep->peers != nullptr)) return MSK_ERR_INVALID;
    if (q->s1 > 1 && (!q->h1_part || !q->route_pub)) return MSK_ERR_INVALID;  // only the K-split gemm 1 leaves FP32 partials
    const int P = q->T * q->top_k;
    if (q->T < 1 || q->top_k < 1 || q->top_k > 8 || P > kMaxPairs || q->local_count < 1 || q->local_count > kMaxExperts ||
        q->T > kMaxPairs / 8)
        return MSK_ERR_UNSUPPORTED;
    if (q->H % 128 != 0 || q->I % 128 != 0 || q->ldx % 8 != 0 || q->H > 16 * kCombineThreads) return MSK_ERR_UNSUPPORTED;
    if (q->logits != nullptr && (q->n_logits > 256 || q->n_logits < q->top_k)) return MSK_ERR_UNSUPPORTED;
    const MskEpHooks* ep = q->ep;
    if (ep != nullptr && ep->peers != nullptr && (ep->n_peers < 1 || ep->rows_per_peer < 1 || ep->done_counter == nullptr || !q->out_fp32))
        return MSK_ERR_INVALID;
    const int direct = q->T <= kGroup;
    // the GEMM reads x itself only when it is FP16 and needs no gathering (and no wait for other GPUs' rows)
    const int stage = !(direct && q->x_fp16) || (ep != nullptr && ep->wait_flags != nullptr);
    if (stage && q->x_sorted == nullptr) return MSK_ERR_INVALID;
    const int s1 = q->s1 > 0 ? q->s1 : 1, s2 = q->s2 > 0 ? q->s2 : 1;
    if ((q->H / 128) % s1 != 0 || (q->I / 128) % s2 != 0) return MSK_ERR_INVALID;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return MSK_ERR_CUDA;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int smem = 1024 + kNRaw * kStage;
    static bool configured[kMaxDevices] = {};  // the attribute is per device
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(moe_gemm_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess ||
            cudaFuncSetAttribute(moe_gemm_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return MSK_ERR_CUDA;
        configured[dev] = true;
    }
    RouteArgs ra{};
    ra.ids = q->topk_ids, ra.logits = q->logits, ra.n_logits = q->n_logits;
    ra.ld_logits = q->ld_logits > 0 ? q->ld_logits : q->n_logits;
    ra.ids_out = q->topk_ids, ra.wts_out = q->topk_weights;
    ra.ld_ids = q->ld_topk > 0 ? q->ld_topk : q->top_k;
    ra.T = q->T, ra.top_k = q->top_k, ra.local_start = q->local_start, ra.local_count = q->local_count;

    // B operands by TMA (FP16, box = 32 rows x 64 k): gemm 1 reads the staged copy of x (tokens as rows up to 32
    // tokens, else rows gathered in expert-list order) or x itself; gemm 2 reads the activations in that order.
    CUtensorMap tm_b1, tm_b2;
    int rc = !stage    ? make_tmap_bf16_kgroups(&tm_b1, q->x, q->T, q->H, q->ldx, kGroup, 4)
             : direct ? make_tmap_bf16_kgroups(&tm_b1, q->x_sorted, q->T, q->H, q->H, kGroup, 4)
                      : make_tmap_bf16_kgroups(&tm_b1, q->x_sorted, P, q->H, q->H, kGroup, 4);
    if (rc == 0) rc = make_tmap_bf16_kgroups(&tm_b2, q->inter_sorted, P, q->I, q->I, kGroup, 4);
    if (rc != 0) return rc;

    int pdl = q->pdl;
    if (stage) {
        MoeStageArgs g{};
        g.route = ra, g.x = q->x, g.ldx = q->ldx, g.H = q->H, g.x_fp16 = q->x_fp16, g.direct = direct;
        g.x16 = static_cast<__half*>(q->x_sorted), g.status = status;
        if (ep != nullptr && ep->wait_flags != nullptr) {
            g.wait_flags = ep->wait_flags, g.wait_count = ep->wait_count, g.wait_value = ep->wait_value;
            g.wait_cycles = ep->wait_cycles > 0 ? ep->wait_cycles : kWaitBudgetCycles;
        }
        const int rows = direct ? q->T : P;
        rc = launch_pdl(moe_stage_kernel, dim3(rows < sms ? rows : sms), dim3(kRouteThreads), 0, s, pdl, g);
        if (rc != 0) return rc;
        pdl = 1;
    }
    MoeGemmArgs a{};
    a.route = ra;
    a.wpacked = static_cast<const uint8_t*>(q->w13_packed), a.gs = q->w13_gs, a.R = 2 * q->I, a.K = q->H, a.direct = direct;
    a.x_ssq = q->x_ssq, a.x_ssq_parts = q->x_ssq_parts, a.x_inv_dim = q->x_inv_dim, a.x_eps = q->x_eps;
    a.x_ssq_ts = q->x_ssq_tstride > 0 ? q->x_ssq_tstride : 1;
    a.route_pub = q->route_pub, a.outp = q->h1_part, a.S = s1, a.status = status;
    a.inter = static_cast<__half*>(q->inter_sorted), a.inner = q->I, a.fuse_act = s1 == 1;
    // the staging kernel precedes: the ids are final, unless they arrive from other GPUs during that kernel
    a.route_early = stage && q->logits == nullptr && !(ep != nullptr && ep->wait_flags != nullptr);
    // compact tables where the build is on the critical path: gemm 1 straight after the kernel that chose the experts
    a.small = direct && q->logits == nullptr && a.fuse_act && !a.route_early;
    a.share_chunks = q->T <= 4;
    rc = launch_pdl2(moe_gemm_kernel<1>, dim3(sms), dim3(kMoeThreads), smem, s, pdl, tm_b1, a);
    if (rc != 0) return rc;

    if (!a.fuse_act) {
        MoeActArgs act{};
        act.route_pub = q->route_pub, act.h1 = q->h1_part, act.s1 = s1, act.P = P, act.inner = q->I;
        act.inter = static_cast<__half*>(q->inter_sorted);
        rc = launch_pdl(moe_act_kernel, dim3(P < 2 * sms ? P : 2 * sms), dim3(256), 0, s, 1, act);
        if (rc != 0) return rc;
    }

    MoeGemmArgs b{};
    b.route = ra;
    b.route.logits = nullptr;  // gemm 1 has published the ids
    b.route.ids_out = nullptr, b.route.wts_out = nullptr;
    b.wpacked = static_cast<const uint8_t*>(q->w2_packed), b.gs = q->w2_gs, b.R = q->H, b.K = q->I, b.direct = 0;
    b.outp = q->y_part, b.S = s2, b.status = status;
    // the ids are final before gemm 2 can start, unless gemm 1 itself chose them from logits and ran just before
    b.route_early = !a.fuse_act || q->logits == nullptr;
    b.share_chunks = a.share_chunks;
    rc = launch_pdl2(moe_gemm_kernel<2>, dim3(sms), dim3(kMoeThreads), smem, s, 1, tm_b2, b);
    if (rc != 0) return rc;

    MoeCombineArgs c{};
    c.ids = q->topk_ids, c.wts = q->topk_weights, c.top_k = q->top_k, c.local_start = q->local_start;
    c.ld_ids = ra.ld_ids;
    c.local_count = q->local_count, c.H = q->H, c.S = s2, c.P = P, c.yp = q->y_part, c.gs = q->w2_gs;
    c.post_w = static_cast<const __nv_bfloat16*>(q->post_norm_w), c.eps = q->post_eps, c.resid = q->resid, c.ldr = q->ldr;
    c.out = q->out, c.out_fp32 = q->out_fp32, c.ldo = q->ldo;
    c.out_copy = static_cast<__nv_bfloat16*>(q->out_copy), c.ldc = q->ldc;
    if (ep != nullptr && ep->peers != nullptr) {
        c.peers = ep->peers, c.n_peers = ep->n_peers, c.rows_per_peer = ep->rows_per_peer, c.out_off = ep->out_off;
        c.flag_off = ep->flag_off, c.flag_value = ep->flag_value, c.done_counter = ep->done_counter;
    }
    if (q->H <= 2 * kCombineThreads * 4 && s2 == 1) return launch_pdl(moe_combine_kernel<2, 1>, dim3(q->T), dim3(kCombineThreads), 0, s, 1, c);
    if (q->H <= 2 * kCombineThreads * 4 && s2 == 2) return launch_pdl(moe_combine_kernel<2, 2>, dim3(q->T), dim3(kCombineThreads), 0, s, 1, c);
    if (q->H <= 2 * kCombineThreads * 4) return launch_pdl(moe_combine_kernel<2, 0>, dim3(q->T), dim3(kCombineThreads), 0, s, 1, c);
    return launch_pdl(moe_combine_kernel<4, 0>, dim3(q->T), dim3(kCombineThreads), 0, s, 1, c);
}

// ---------------------------------------------------------------- routed experts without caller scratch
// Some hosts cannot hand this library scratch memory and cannot let it allocate either: an inference
// server whose memory pool claimed the whole device at start-up (any later cudaMalloc fails or fragments
// its arena), or a step that is already inside a latency-critical loop where an allocation would
// synchronise the device.  For them all the scratch of msk_moe_forward (the FP32 partials, the activations between the GEMMs,
// the routing list) lives in the array
// below, which every GPU that loads the library holds until the process exits.
// Limit: everything msk_moe_scratch_bytes reports for the call, each part rounded up to 256 bytes, must fit
// in 4 MiB (e.g. 8 tokens at the benchmark's expert shapes with s1 = 4, s2 = 2).
constexpr size_t kStaticScratchFloats = 1u << 20;
static __device__ __align__(256) float g_moe_static_scratch[kStaticScratchFloats];

namespace {
float* g_static_scratch_ptr[msk::kMaxDevices] = {};  // device address of the array, per device
}  // namespace

extern "C" int msk_moe_forward_static(const MskMoeParams* q, int* status, void* stream) {
    if (q == nullptr) return MSK_ERR_INVALID;
    const size_t s1 = q->s1 > 0 ? q->s1 : 1, s2 = q->s2 > 0 ? q->s2 : 1;
    if (q->T < 1 || q->top_k < 1 || q->H < 1 || q->I < 1) return MSK_ERR_INVALID;
    size_t part[5];
    if (msk_moe_scratch_bytes(q->T, q->top_k, q->H, q->I, static_cast<int>(s1), static_cast<int>(s2), &part[0], &part[1], &part[2],
                              &part[3], &part[4]) != 0)
        return MSK_ERR_INVALID;
    size_t off[5], total = 0;
    for (int i = 0; i < 5; ++i) {
        off[i] = total;
        total += (part[i] + 255) / 256 * 256;
    }
    if (total > kStaticScratchFloats * sizeof(float)) return MSK_ERR_UNSUPPORTED;  // beyond the built-in scratch
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= msk::kMaxDevices) return MSK_ERR_CUDA;
    if (g_static_scratch_ptr[dev] == nullptr) {
        // Set-up, once per device and with that device current.  In host code the array's name is only a
        // stand-in; kernels need the address the runtime reports for the symbol on this device.
        float* p = nullptr;
        if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_moe_static_scratch) != cudaSuccess || p == nullptr)
            return MSK_ERR_CUDA;
        g_static_scratch_ptr[dev] = p;
    }
    MskMoeParams m = *q;
    char* basep = reinterpret_cast<char*>(g_static_scratch_ptr[dev]);
    m.h1_part = reinterpret_cast<float*>(basep + off[0]);
    m.y_part = reinterpret_cast<float*>(basep + off[1]);
    m.inter_sorted = basep + off[2];
    m.x_sorted = part[3] ? basep + off[3] : nullptr;
    m.route_pub = reinterpret_cast<int32_t*>(basep + off[4]);
    return msk_moe_forward(&m, status, stream);
}

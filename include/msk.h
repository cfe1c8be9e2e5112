/* C ABI of libmsk_b200.so: one decoder layer's decode step on B200 (sm_100a).
 *
 * Every entry point takes plain device pointers and sizes, launches on the given CUDA stream
 * (a cudaStream_t passed as void*), never synchronises and never allocates: every buffer, scratch
 * included, is the caller's (the *_bytes functions give the sizes).  Return value: 0 on success, a
 * negative code for a rejected call (-1 invalid argument, -2 CUDA error, -3 unsupported shape).
 * Device-side problems (a bounded wait that expired, an index out of range) do not trap: the
 * kernel records them in `status`, a device int32[4] owned by the caller:
 *   status[0] code (1 timeout, 2 bounds, 3 capacity), status[1] kernel<<8|site, status[2..3] detail.
 * The caller zeroes it once and reads it back outside any timed region.
 *
 * Each function names the interface of the reference (Kushagrabainsla/muse-spark-open) that it
 * stands in for, by path inside that project.
 */
#ifndef MSK_H
#define MSK_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

int msk_version(void);

/* Number of SMs / L2 bytes of the current device (for sizing flush buffers and grids). */
int msk_device_info(int* sm_count, int* l2_bytes);

/* Layout self-test of one tensor-core operand path on a toy product (see csrc/selftest.cu).
 * Replaces the reference's tools/wg_test.py (muse_attention_decode/tools/wg_test.py:39-126),
 * which validates MMA descriptor and fragment layouts on a 64x64 toy before the real kernel. */
int msk_selftest_umma(int mode, const void* a, const void* b, float* d, int n, int* status, void* stream);

/* ---------------------------------------------------------------- skinny BF16 projection
 * out[M, N] = x[M, K] * W[N, K]^T with FP32 accumulation, M <= 256, K % 64 == 0.
 * Stands in for muse_bf16_proj/submission.py: `skinny` (pybind, :316-325) / `skinny_kernel`
 * (:161-286) behind `kernel_fn` (:416-436), including the layer hooks `data["out"]` (ldo) and
 * `data["ssq"]` (out_ssq) of :430-435.
 *
 * Optional fused epilogue, applied in this order to the FP32 accumulator acc[t, n]:
 *   acc *= rsqrt(sum_p in_ssq[p*M + t] * in_inv_dim + in_eps)   (RMSNorm of the input rows, folded)
 *   acc += resid[t*ldr + n]                                       (FP32 residual)
 *   out (bf16 or fp32) = acc
 *   out_normed[t*ldn + n] = bf16 or fp16(acc * (1 + next_norm_w[n]))   (input of the next op, un-normalised)
 *   out_ssq[tile*M + t] = sum over the tile's 128 columns of acc^2 (tile = n / 128)
 */
typedef struct {
    const void* x;          /* bf16 [M, K], row stride K */
    const void* w;          /* bf16 [N, K], row stride K */
    int M, N, K;
    int splits;             /* split-K ways, 1..16; 0 = pick so that tiles x splits fills the device */
    int token_splits;       /* CTAs sharing the tokens of a tile, 1..16; 0 = pick (more than one from 128 tokens up) */
    void* out;              /* [M, ldo] bf16, or fp32 when out_fp32 != 0; may be NULL */
    int out_fp32;
    int ldo;
    const float* in_ssq;    /* [in_ssq_parts, M] partial sums of squares of the un-normalised input, or NULL */
    int in_ssq_parts;
    float in_inv_dim;
    float in_eps;
    const float* resid;     /* fp32 [M, ldr] or NULL */
    int ldr;
    const void* next_norm_w;/* bf16 [N] or NULL */
    void* out_normed;       /* bf16 (fp16 when normed_fp16 != 0) [M, ldn] or NULL */
    int ldn;
    float* out_ssq;         /* fp32 [ceil(N/128), M] or NULL */
    int pdl;                /* launch with programmatic stream serialization (the kernel waits for its
                               predecessor only after it has started streaming W) */
    int normed_fp16;        /* out_normed is written as FP16 (saturating), what the experts' GEMM consumes */
    void* scratch;          /* split-K workspace, msk_proj_scratch_bytes() bytes, 16-byte aligned: tile tickets (its
                               first 4096 bytes, zero before the first launch; every launch leaves them zero) and
                               the FP32 partial tiles.  May be NULL when the launch runs unsplit.  Launches that may
                               overlap on the GPU need a workspace each. */
    size_t scratch_bytes;
} MskProjParams;

int msk_proj_skinny(const MskProjParams* p, int* status, void* stream);

/* Bytes of the split-K workspace for a launch of that shape on the current device (splits and token_splits as
 * in MskProjParams).
 * Stands in for the reference's per-(layer, m) split table (muse_bf16_proj/submission.py:288-314,352-364),
 * whose partials live in distributed shared memory instead. */
int msk_proj_scratch_bytes(int M, int N, int K, int splits, int token_splits, size_t* bytes);

/* ---------------------------------------------------------------- gated attention decode / verify
 * One decode step (L = 1) or one 8-token verify block (L = 8, causal inside the block) of gated
 * attention over a paged FP8-E4M3 KV cache: per-head RMSNorm of q and k, q * qk_scale_factor,
 * interleaved RoPE, the new tokens' K/V quantised and written into the cache at `cache_loc`,
 * softmax(q.k * sm_scale) over the visible keys (sliding window: a token and the window-1 before it;
 * window 0 = all), output RMSNorm per head times sigmoid(gate), BF16.
 * Stands in for muse_attention_decode/submission.py `kernel_fn` (:2363-2372) and the kernels behind it
 * (`attnc_kernel` :1604-1856, `attnpcc_kernel` :1915-2284, `attn_kernel` + `_prep` + `_attn_combine`
 * :293-539,115-173); the fields mirror its `Inputs` / `Config` (:37-65).
 * Built for head_dim 128, Hq = 8 * Hkv, page_size a power of two in [8, 128].
 */
typedef struct {
    const void* qkv;          /* bf16 [B*L, ld_qkv]: q (Hq*d) | k (Hkv*d) | v (Hkv*d) | gate (Hq*d) per token */
    int ld_qkv;
    void* out;                /* bf16 [B*L, ld_out], Hq*d values per token */
    int ld_out;
    void* k_cache;            /* e4m3 [num_pages, page_size, Hkv, d], new rows written in place */
    void* v_cache;
    const float* k_scale;     /* device scalars: value = e4m3 * scale */
    const float* v_scale;
    const int32_t* seq_lens;  /* [B] cached tokens per request; the block starts at this position */
    const int32_t* page_table;/* [B, max_pages] physical page of each logical page, -1 = none */
    int max_pages;
    const int64_t* cache_loc; /* [B*L] flat cache row (page * page_size + slot) of each new token */
    const float* inv_freq;    /* [d/2] RoPE frequencies theta^(-2i/d) as FP32, or NULL for no RoPE */
    int B, L, Hq, Hkv, d, page_size, num_pages, window;
    float qk_scale_factor, sm_scale;
    int chunks;               /* split-KV ways = cluster size (1, 2, 4 or 8); 0 = pick */
    int stages;               /* K/V tile ring depth (3 to 6, as far as shared memory allows); 0 = pick: 3 for decode, 4 for verify */
    int issuers;              /* MMA-issuing warps beside the arithmetic warps: 1; 0 = pick */
    int pdl;
    int row_groups;           /* sets of four arithmetic warps that split the 8 L query rows of a KV head: 2 (decode), 4 (verify); 0 = pick */
} MskAttnParams;

int msk_attn_decode(const MskAttnParams* p, int* status, void* stream);

/* ---------------------------------------------------------------- NVFP4 (w4a16) routed experts
 * Per local (token, slot) pair: h = x . W13[e]^T, inter = fp16(silu(h[:I]) * h[I:]), y = inter . W2[e]^T,
 * out[token] += topk_weight * rmsnorm(y * (1 + post_norm_w), eps); tokens without a local pair give zeros.
 * Weights are NVFP4: E2M1 codes (two per byte, low nibble first), one E4M3 scale per 16 values, one FP32
 * scale per expert.  Stands in for muse_moe_w4a16/submission.py: `prepare` + `_pack_expert` (:793-871),
 * `moe_forward` (pybind, :730-768) behind `kernel_fn` (:874-897) = `moe_gemm` x2 + `norm_kernel`
 * (:307-666), with the layer hooks `pre_norm` (x_ssq) and `local_start_dev` of :888-896.
 * The tensor cores run FP16 x FP16 -> FP32: the dequantised weights (E2M1 x E4M3) are exact in FP16, a BF16
 * activation converts exactly for 2^-14 <= |x| <= 65504 (smaller magnitudes round to multiples of 2^-24).
 */
typedef struct {
    const void* w13;     /* uint8 [E, 2I, H/2]: gate rows [0, I) then up rows [I, 2I) */
    const void* w13_sf;  /* e4m3  [E, 2I, H/16] */
    const void* w2;      /* uint8 [E, H, I/2] */
    const void* w2_sf;   /* e4m3  [E, H, I/16] */
    int E, H, I;         /* H and I multiples of 128 */
} MskMoeWeights;

/* Bytes of the two repacked weight buffers (lossless: same codes and scales, re-ordered into 9216-byte
 * blocks of 128 rows x 128 k; in W13 every 32 rows of a block are 16 gate rows and the 16 up rows of the same
 * channels). */
int msk_moe_packed_bytes(int E, int H, int I, size_t* w13_bytes, size_t* w2_bytes);
int msk_moe_pack(const MskMoeWeights* w, void* w13_packed, void* w2_packed, void* stream);
/* Test hook: expand a packed buffer to BF16 [E, R, K] = e2m1 * e4m3 scale (no per-expert scale), rows in the
 * original order; gate_up != 0 for a packed W13 (R = 2I). */
int msk_moe_dequant(const void* packed, void* out_bf16, int E, int R, int K, int gate_up, void* stream);
/* Bytes of the scratch buffers msk_moe_forward needs for T tokens (h1 and route only with s1 > 1). */
int msk_moe_scratch_bytes(int T, int top_k, int H, int I, int s1, int s2, size_t* h1_bytes, size_t* y_bytes,
                          size_t* inter_bytes, size_t* x_sorted_bytes, size_t* route_bytes);

/* Hooks that turn msk_moe_forward into one rank's share of the expert-parallel step (see msk_ep_step): the
 * input rows arrive from other GPUs (the first kernel waits for their flags) and every token's partial result
 * row is stored straight into its home GPU's memory; when all rows are written the last block sets a flag in
 * every peer.  No counterpart in the reference (one GPU, collectives stated as identities,
 * muse_decode_layer/reference.py:8-10). */
typedef struct {
    const int32_t* wait_flags;  /* local device int32[wait_count]; the first kernel waits (bounded) until each >= wait_value */
    int wait_count, wait_value;
    long long wait_cycles;      /* budget of one wait in SM clocks; 0 = about half a second */
    void* const* peers;         /* device array [n_peers] of the peers' regions as mapped on this GPU; NULL = rows stay local */
    int n_peers, rows_per_peer; /* token t is at home on peer t / rows_per_peer */
    size_t out_off;             /* byte offset, inside a peer's region, of this rank's block of FP32 rows [rows_per_peer, ldo] */
    size_t flag_off;            /* byte offset of the int32 this rank sets to flag_value in every peer's region at the end */
    int flag_value;
    int32_t* done_counter;      /* local device int32, zero before the first call (left zero by every call) */
} MskEpHooks;

typedef struct {
    const void* x;              /* [T, ldx] bf16, or fp16 when x_fp16 != 0 */
    int ldx;
    const float* x_ssq;         /* optional: [x_ssq_parts, T] partial sums of squares of the un-normalised */
    int x_ssq_parts;            /*   rows; gemm 1 then scales row t by rsqrt(sum * x_inv_dim + x_eps)      */
    float x_inv_dim, x_eps;
    int32_t* topk_ids;          /* [T, top_k] global expert ids: input, or output when logits != NULL */
    float* topk_weights;        /* [T, top_k] */
    int ld_topk;                /* ints (floats) between token rows of topk_ids / topk_weights; 0 = top_k */
    const float* logits;        /* optional [T, n_logits]: softmax -> top-k -> renormalise inside the GEMM CTAs */
    int n_logits;
    int ld_logits;              /* floats between token rows of logits; 0 = n_logits */
    int x_ssq_tstride;          /* floats between tokens inside one part of x_ssq; 0 = 1 (parts are T*stride apart) */
    int T, top_k;               /* T <= 256, top_k <= 8 */
    int local_start, local_count; /* this GPU holds experts [local_start, local_start + local_count) */
    const void* w13_packed;
    const void* w2_packed;
    const float* w13_gs;        /* [local_count] */
    const float* w2_gs;
    const void* post_norm_w;    /* bf16 [H] */
    float post_eps;
    int H, I;
    float* h1_part;             /* scratch fp32 [s1, T*top_k, 2I]; only needed for s1 > 1 */
    float* y_part;              /* scratch fp32 [s2, T*top_k, H]: the down projections' sums before the experts' global scales (the combine kernel applies them) */
    void* inter_sorted;         /* scratch fp16 [T*top_k, I]: activations between the GEMMs, expert-list order */
    void* x_sorted;             /* scratch fp16: [T, H] up to 32 tokens, else [T*top_k, H] (inputs gathered in
                                   expert-list order); not needed for T <= 32 with x_fp16 */
    int32_t* route_pub;         /* scratch int32 [2 + T*top_k]: the routing list gemm 1 publishes; only for s1 > 1 */
    int s1, s2;                 /* K splits of the two GEMMs (divide H/128 and I/128); 0 = 1.  With s1 = 1 the
                                   activation is applied in gemm 1's epilogue (one launch fewer) */
    const float* resid;         /* optional fp32 [T, ldr] added to the result */
    int ldr;
    void* out;                  /* [T, ldo] bf16, or fp32 when out_fp32 != 0 */
    int out_fp32, ldo;
    void* out_copy;             /* optional bf16 [T, ldc] copy of the result */
    int ldc;
    int pdl;
    int x_fp16;                 /* x is FP16 already (the layer's o_proj epilogue writes it so) */
    const MskEpHooks* ep;       /* expert-parallel hooks (host pointer, read during the call); NULL = single GPU */
} MskMoeParams;

int msk_moe_forward(const MskMoeParams* p, int* status, void* stream);

/* msk_moe_forward for callers that can neither pass scratch nor let the library allocate (a server whose
 * memory pool owns the whole device, a step inside a loop where an allocation would stall the GPU).
 * No counterpart in the reference, whose kernel_fn allocates freely (muse_moe_w4a16/submission.py:882-886).
 * The scratch pointers of `p` are ignored: all scratch lives in a 4 MiB array inside the library that each
 * GPU holds from load to exit.  Accepted while the five sizes msk_moe_scratch_bytes reports for the call,
 * each rounded up to 256 bytes, sum to at most 4 194 304 bytes (8 tokens at the benchmark's expert shapes
 * with s1 = 4, s2 = 2); larger calls return -3 and run nothing.
 * It calls no cudaMalloc / cudaFree and nothing that allocates.  The first call on a device looks up the
 * array's device address (cudaGetSymbolAddress): make that call before any stream capture.  All calls
 * on a device share the array; nothing in it has to be zero on entry and it keeps the last call's
 * partials, so two calls whose kernels overlap on the GPU (different streams) race: run them in order. */
int msk_moe_forward_static(const MskMoeParams* p, int* status, void* stream);

/* ---------------------------------------------------------------- whole decoder layer, decode step
 * stream fp32 [T, H] -> input RMSNorm -> fused QKV+gate projection -> gated attention over the paged
 * FP8 cache (new K/V written in place) -> o_proj + residual -> pre-expert RMSNorm -> FP32 router
 * (softmax top-k renormalised, chosen inside the expert GEMM CTAs) -> NVFP4 experts, post-expert norm,
 * weighted sum -> + residual.  T = B * L tokens.  Eight kernels chained with programmatic dependent
 * launch; both RMSNorms are folded (row scale from sums of squares the producing kernel leaves).
 * Stands in for muse_decode_layer/submission.py `kernel_fn` (:3978-4038) on the op list the benchmark
 * names; `prepare` (same file) corresponds to msk_moe_pack plus buffer allocation by the caller.
 *
 * msk_layer_front runs everything up to the router's expert choice (what an expert-parallel rank does before
 * the token exchange); msk_layer_decode adds the experts and the second residual on one GPU.
 */
typedef struct {
    int B, L, H, Hq, Hkv, d, page_size, num_pages, max_pages, window;
    float qk_scale_factor, sm_scale, norm_eps;
    const float* stream;           /* fp32 [T, H] residual stream in */
    /* attention step metadata and cache, as MskAttnParams */
    void* k_cache;
    void* v_cache;
    const float* k_scale;
    const float* v_scale;
    const int32_t* seq_lens;
    const int32_t* page_table;
    const int64_t* cache_loc;
    const float* inv_freq;
    /* weights */
    const void* input_norm_w;      /* bf16 [H] (scale = 1 + w) */
    const void* w_qkv;             /* bf16 [(2Hq+2Hkv)*d, H] */
    const void* w_o;               /* bf16 [H, Hq*d] */
    const void* pre_expert_norm_w; /* bf16 [H] */
    const float* router_w;         /* fp32 [E, H] */
    const float* router_bias;      /* fp32 [E] or NULL */
    int E;
    /* scratch owned by the caller (allocated once) */
    void* xn0;                     /* bf16 [T, H] */
    float* ssq0;                   /* fp32 [T] */
    void* qkv;                     /* bf16 [T, (2Hq+2Hkv)*d] */
    void* attn;                    /* bf16 [T, Hq*d] */
    float* stream1;                /* fp32 [T, H] stream after attention */
    void* xn1;                     /* fp16 [T, H] expert input before its row scale */
    float* ssq1;                   /* fp32 [H/128 + 1, T]: per-128-column partial sums of squares, last row their total */
    float* router_part;            /* fp32 [H/128, T, E] */
    int32_t* router_ticket;        /* int32 [ceil(T/32) * (ceil(E/32) + 1)], zero before the first call */
    void* qkv_scratch;             /* split-K workspaces of the two projections (msk_proj_scratch_bytes for   */
    void* o_scratch;               /*   [T, (2Hq+2Hkv)*d, H] and [T, H, Hq*d]), first 4096 bytes zero before the */
    size_t qkv_scratch_bytes, o_scratch_bytes; /* first call */
    float* logits;                 /* fp32 [T, E] */
    int top_k;                     /* <= 8 */
    int32_t* topk_ids;             /* int32 [T, top_k]: softmax -> top-k -> renormalise of the logits, written by */
    float* topk_weights;           /* fp32 [T, top_k]    the router kernel's last block per 32 tokens */
    int attn_chunks, attn_stages, attn_issuers, qkv_splits, o_splits;
    int attn_row_groups;
    int pdl;                       /* also chain the first kernel to whatever precedes it */
} MskLayerFront;

int msk_layer_front(const MskLayerFront* p, int* status, void* stream);

typedef struct {
    MskLayerFront front;
    MskMoeParams moe;              /* x, x_ssq, topk_ids, topk_weights, top_k, resid, T, H are filled from `front` */
} MskLayerParams;

int msk_layer_decode(const MskLayerParams* p, int* status, void* stream);

/* ---------------------------------------------------------------- pieces of the reference's own layer form
 * The reference's layer (muse_decode_layer/reference.py:447-477) differs from the benchmark's op list in its
 * residual boundaries (norm-preserving gated mixes, :339-344), its routing rule (sigmoid scores chosen by score +
 * bias, :419-424) and a pooler / unpooler pair of projections around the experts.  These entry points are those
 * pieces; muse_spark_open_b200/layer.py::native_kernel_fn chains them with msk_proj_skinny, msk_attn_decode and
 * msk_moe_forward.
 */
typedef struct {
    const float* x;              /* fp32 [T, H]: rows before their RMSNorm (the stream after attention) */
    const void* norm_w;          /* bf16 [H]: the router sees rmsnorm(x, eps) * (1 + norm_w), in FP32 */
    float* ssq;                  /* fp32 [ssq_parts + 1, T]: partial sums of squares of the rows (in); the last row
                                    receives their totals (out) */
    int ssq_parts;
    float eps;
    const float* router_w;       /* fp32 [E, H] */
    const float* router_bias;    /* fp32 [E] or NULL */
    int E, T, H, top_k;          /* H a multiple of 1024, <= 8192; E <= 256; top_k <= 8 */
    int sigmoid_bias;            /* 0: softmax(logits + bias), top-k, renormalise; 1: sigmoid(multiplier * logit), top-k
                                    of score + bias, weights = scores / (sum + 1e-15) */
    float multiplier;
    float* part;                 /* scratch fp32 [H/128, T, E] */
    int32_t* ticket;             /* scratch int32 [ceil(T/32) * (ceil(E/32) + 1)], zero before the first call */
    float* logits;               /* fp32 [T, E] (without the bias when sigmoid_bias) */
    int32_t* topk_ids;           /* int32 [T, top_k] */
    float* topk_weights;         /* fp32 [T, top_k] */
    int pdl;
} MskRouterParams;

/* FP32 router: logits on CUDA cores (expert ids must not depend on tensor-core rounding), then the expert choice.
 * Stands in for the router GEMM + routing kernel of muse_decode_layer/submission.py:3998-4016. */
int msk_router(const MskRouterParams* p, int* status, void* stream);

typedef struct {
    const float* stream;         /* fp32 [T, H] */
    const void* branch;          /* [T, ldb] fp32, or bf16 when branch_bf16 != 0 */
    int branch_bf16, ldb;
    const void* branch_w;        /* bf16 [H] or NULL: the branch is scaled by (1 + branch_w) first */
    const void* gate;            /* bf16 [H] residual gate, or NULL for a plain add */
    const void* next_norm_w;     /* bf16 [H] or NULL */
    float* stream_out;           /* fp32 [T, H] or NULL */
    void* normed_out;            /* bf16 [T, H] = rmsnorm(stream_out, eps) * (1 + next_norm_w), or NULL */
    float* ssq_out;              /* fp32 [T] sums of squares of stream_out, or NULL */
    int T, H;                    /* H a multiple of 4, <= 8192 */
    float branch_eps, eps, temperature, gate_eps;
    int pdl;
} MskBoundaryParams;

/* stream_out = alpha * stream + beta * rmsnorm(branch * (1 + branch_w), branch_eps) with
 * beta = sigmoid(gate / temperature), alpha = sqrt(max(sigmoid(-gate / temperature) * (1 + beta), gate_eps))
 * (muse_decode_layer/reference.py:339-344,452-455,473-476: the SGLang residual-boundary kernels of the reference's
 * submission have no source in its tree; this follows ref_front / ref_back). */
int msk_residual_boundary(const MskBoundaryParams* p, void* stream);

/* out = bf16(rmsnorm(x, eps) * (1 + w)), ssq[t] = sum x[t]^2 (the pre-expert norm after the pooler,
 * muse_decode_layer/reference.py:465). */
int msk_rmsnorm(const float* x, const void* w, void* out_bf16, float* ssq, int T, int H, float eps, int pdl, void* stream);

/* ---------------------------------------------------------------- expert-parallel step
 * The reference runs one GPU and states its collectives as identities (muse_decode_layer/reference.py:8-10,
 * :467 "the all-reduce: identity"); here the exchange is real.  Requests are data-parallel (rank r owns T_local
 * tokens), experts expert-parallel (rank r holds experts [r*E/world, (r+1)*E/world)), dense weights replicated.
 *
 * Device-initiated exchange (msk_ep_step): every rank owns one "region" of device memory that all peers map
 * (CUDA IPC).  Per step, with buffers chosen by the parity of the step number:
 *   dispatch   a kernel packs each local token's row (expert input fp16 | expert ids | weights | sum of squares)
 *              and stores it into EVERY peer's region (plain stores over NVLink); the last block sets
 *              dispatch_flag[rank] = step in every peer.
 *   experts    msk_moe_forward over all world * T_local rows of the own region with the local experts; its first
 *              kernel waits (bounded) for every source's dispatch flag; the combine kernel stores each token's
 *              weighted, post-normed partial row into the token's home region (tokens without a local expert
 *              send nothing) and finally sets combine_flag[rank] = step in every peer.
 *   reduce     waits (bounded) for every rank's combine flag, then out[t] = stream1[t] + the partial rows of the
 *              ranks that hold one of the token's experts, added in rank order (bitwise reproducible).
 * No collective library call, no host synchronisation; an expired wait records MSK_ERR_TIMEOUT in `status` and
 * the kernels run to their end.  A buffer is reused two steps later, by which time every reader is done (a rank
 * starts step s only after its reduce of step s - 1, which needed every peer's combine of step s - 1).
 *
 * Region layout (msk_ep_region_bytes): int32 dispatch flags [2][64] | int32 combine flags [2][64] |
 * rows uint8 [2][world * T_local][row_bytes] | partials fp32 [2][world][T_local][H].
 */
int msk_ep_row_bytes(int H, int top_k); /* 2H (x, 2-byte elements) + 4k ids + 4k weights (padded to 16) + 16 (sum of squares, padding) */
int msk_ep_region_bytes(int world, int T_local, int H, int top_k, size_t* bytes);

/* Set-up helpers, the only entry points of this library that allocate or map memory: a zeroed region from
 * cudaMalloc with its 64-byte CUDA IPC handle; a peer's region opened from its handle; their release. */
int msk_ep_region_alloc(size_t bytes, void** ptr, void* handle64);
int msk_ep_region_open(const void* handle64, void** ptr);
int msk_ep_region_close(void* ptr);
int msk_ep_region_free(void* ptr);

typedef struct {
    int rank, world, T_local, n_experts;
    int step;                  /* 1, 2, 3, ...: the same on every rank, one more each call */
    void* self;                /* this rank's region */
    void* const* peers;        /* device array [world]: every rank's region as mapped on this GPU (peers[rank] = self) */
    int32_t* counters;         /* local device int32[2], zero before the first step */
    long long wait_cycles;     /* budget of one wait for a peer's flag, SM clocks; 0 = about half a second */
} MskEpComm;

typedef struct {
    MskLayerFront front;       /* this rank's requests up to the router's expert choice */
    MskMoeParams moe;          /* local experts and scratch for world * T_local tokens; x, ids, weights, x_ssq, T, resid,
                                  out and ep are filled in from `comm` */
    MskEpComm comm;
    float* out;                /* fp32 [T_local, H] stream after the layer */
    void* hidden;              /* bf16 [T_local, H] copy, or NULL */
} MskEpStep;

int msk_ep_step(const MskEpStep* p, int* status, void* stream);

/* The same step's kernels for an exchange done by a collective library instead (NCCL all-gather of the rows,
 * all-to-all of the partials): rows packed by msk_ep_pack, msk_moe_forward over the gathered rows, msk_ep_reduce
 * adds the ranks' partials to the residual in rank order. */
int msk_ep_pack(const void* xn, const int32_t* topk_ids, const float* topk_weights, const float* ssq, int ssq_parts,
                void* rows, int T, int H, int top_k, void* stream);
int msk_ep_reduce(const float* stream1, const float* recv /* [ranks, T, H] */, int ranks, float* out, void* out_bf16,
                  int T, int H, void* stream);

/* Test hook for the bounded wait between GPUs: one block waits wait_cycles SM clocks for an int32 flag that
 * nothing sets, must record MSK_ERR_TIMEOUT in status and return (no fault, no hang). */
int msk_selftest_flag_timeout(const int32_t* flag, long long wait_cycles, int* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MSK_H */

// Device-initiated token exchange of the expert-parallel decode step: kernels that store into other GPUs' memory
// over NVLink (plain peer stores through pointers mapped with CUDA IPC; no multicast, no collective library) and
// signal with flags, plus the step's launch chain.
//   ep_dispatch   (home rank) one block per local token: packs the token's row (expert input fp16 | expert ids |
//                 weights | sum of squares) and stores it into every rank's region, its own included; the last block
//                 (ticket) sets dispatch_flag[rank] = step in every region.
//   ep_reduce     (home rank) waits, bounded, for every rank's combine flag; out[t] = stream1[t] + the partial rows
//                 of the ranks that hold one of the token's experts, in rank order.
// The experts in between are msk_moe_forward with its expert-parallel hooks (csrc/moe_nvfp4.cu).
// Flags carry the step number (monotonic), buffers alternate with its parity: nothing is ever reset, and a rank can
// be at most one step ahead of a peer that still reads the other buffer.
#include "msk.h"
#include "ptx.cuh"

namespace msk {

constexpr int kEpMaxWorld = 64;
constexpr size_t kEpFlagBytes = 2 * kEpMaxWorld * sizeof(int);  // one flag array: [2 parities][64 ranks]

struct EpLayout {
    size_t rows_off, recv_off, total;
    int row_bytes;
    __host__ __device__ size_t dflag(int par, int src) const { return (static_cast<size_t>(par) * kEpMaxWorld + src) * sizeof(int); }
    __host__ __device__ size_t cflag(int par, int src) const { return kEpFlagBytes + dflag(par, src); }
};

static EpLayout ep_layout(int world, int T_local, int H, int top_k) {
    EpLayout l;
    l.row_bytes = msk_ep_row_bytes(H, top_k);
    l.rows_off = 2 * kEpFlagBytes;
    const size_t rows = static_cast<size_t>(world) * T_local * l.row_bytes;
    l.recv_off = (l.rows_off + 2 * rows + 255) / 256 * 256;
    l.total = l.recv_off + 2 * static_cast<size_t>(world) * T_local * H * sizeof(float);
    return l;
}

struct EpDispatchArgs {
    const uint16_t* xn;     // [T_local, H] fp16 expert input (un-normalised)
    const int* ids;         // [T_local, top_k]
    const float* wts;
    const float* ssq;       // [T_local] sums of squares of the rows
    void* const* peers;
    int world, rank, T_local, H, top_k, row_bytes, step;
    size_t rows_off;        // byte offset of this step's row buffer inside a region
    size_t flag_off;        // byte offset of dispatch_flag[parity][rank]
    int* counter;
};

__global__ void __launch_bounds__(256) ep_dispatch_kernel(EpDispatchArgs p) {
    const int t = blockIdx.x, tid = threadIdx.x;
    __shared__ uint8_t* peer_s[32];  // the regions' addresses do not depend on the previous kernel: fetched under its tail
    if (tid < p.world) peer_s[tid] = static_cast<uint8_t*>(p.peers[tid]);
    pdl_wait();
    pdl_launch_dependents();
    __syncthreads();
    // the row's pieces are loaded once and stored to every region
    const uint4* src = reinterpret_cast<const uint4*>(p.xn + static_cast<size_t>(t) * p.H);
    const int nv = p.H / 8;  // 16-byte pieces of x
    uint4 v[4];              // H <= 8192
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = tid + 256 * i < nv ? __ldcg(src + tid + 256 * i) : make_uint4(0, 0, 0, 0);
    int id = 0;
    float w = 0.0f, s = 0.0f;
    if (tid < p.top_k) id = __ldcg(p.ids + t * p.top_k + tid), w = __ldcg(p.wts + t * p.top_k + tid);
    if (tid == 32) s = __ldcg(p.ssq + t);
    const size_t row_off = p.rows_off + (static_cast<size_t>(p.rank) * p.T_local + t) * p.row_bytes;
    for (int r0 = 0; r0 < p.world; ++r0) {
        const int r = (r0 + p.rank) % p.world;  // every rank starts with a different peer
        uint8_t* row = peer_s[r] + row_off;
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if (tid + 256 * i < nv) reinterpret_cast<uint4*>(row)[tid + 256 * i] = v[i];
        if (tid < p.top_k) {
            reinterpret_cast<int*>(row + 2 * p.H)[tid] = id;
            reinterpret_cast<float*>(row + 2 * p.H + 4 * p.top_k)[tid] = w;
        }
        if (tid == 32) *reinterpret_cast<float4*>(row + p.row_bytes - 16) = make_float4(s, 0.0f, 0.0f, 0.0f);
    }
    // The block's stores are ordered before the barrier, the barrier before thread 0's fence: one system-scope fence
    // per block covers all of them (256 of them cost the step several microseconds).
    __syncthreads();
    if (tid == 0) {
        __threadfence_system();
        const int old = atomicAdd(p.counter, 1);
        if (old == static_cast<int>(gridDim.x) - 1) {
            *p.counter = 0;
            __threadfence_system();  // every block's rows (each fenced before its ticket) precede the flags
            for (int r = 0; r < p.world; ++r)
                st_relaxed_sys(reinterpret_cast<int*>(peer_s[r] + p.flag_off), p.step);
        }
    }
}

struct EpReduceArgs {
    const float* stream1;   // [T_local, H]
    const int* ids;         // [T_local, top_k] this rank's expert choice
    const float* recv;      // this step's partials [world][T_local][H] in the own region
    const int* flags;       // combine_flag[parity][0..world) in the own region
    int world, T_local, H, top_k, experts_per_rank, step;
    long long wait_cycles;
    float* out;
    __nv_bfloat16* out_bf16;
    int* status;
};

__global__ void __launch_bounds__(256) ep_reduce_peer_kernel(EpReduceArgs p) {
    __shared__ unsigned owners_s;
    const int t = blockIdx.x, tid = threadIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    if (tid == 0) {
        unsigned m = 0;  // ranks that hold one of this token's experts
        for (int k = 0; k < p.top_k; ++k) {
            const int r = __ldcg(p.ids + t * p.top_k + k) / p.experts_per_rank;
            if (r >= 0 && r < p.world && r < 32) m |= 1u << r;
        }
        owners_s = m;
    }
    if (tid >= 32 && tid < 32 + p.world) flag_wait_ge(p.flags + (tid - 32), p.step, p.wait_cycles, p.status, (MSK_K_EP << 8) | 2);
    __syncthreads();
    const unsigned owners = owners_s;
    for (int d = tid * 4; d < p.H; d += 1024) {
        float4 acc = __ldcg(reinterpret_cast<const float4*>(p.stream1 + static_cast<size_t>(t) * p.H + d));
        float4 v[8];
        for (int r0 = 0; r0 < p.world; r0 += 8) {  // eight ranks' loads in flight, added in rank order
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int r = r0 + j;
                v[j] = (r < p.world && ((owners >> r) & 1u))
                           ? __ldcg(reinterpret_cast<const float4*>(p.recv + (static_cast<size_t>(r) * p.T_local + t) * p.H + d))
                           : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (r0 + j < p.world && ((owners >> (r0 + j)) & 1u)) acc.x += v[j].x, acc.y += v[j].y, acc.z += v[j].z, acc.w += v[j].w;
        }
        *reinterpret_cast<float4*>(p.out + static_cast<size_t>(t) * p.H + d) = acc;
        if (p.out_bf16 != nullptr)
            *reinterpret_cast<uint2*>(p.out_bf16 + static_cast<size_t>(t) * p.H + d) =
                make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
    }
}

__global__ void flag_timeout_kernel(const int* flag, long long cycles, int* status) {
    if (threadIdx.x == 0) flag_wait_ge(flag, 0x7fffffff, cycles, status, (MSK_K_EP << 8) | 3);
}

template <typename Args>
static int launch_ep(void (*kern)(Args), int grid, cudaStream_t stream, const Args& a) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, a) == cudaSuccess ? 0 : MSK_ERR_CUDA;
}

}  // namespace msk

extern "C" int msk_ep_region_bytes(int world, int T_local, int H, int top_k, size_t* bytes) {
    using namespace msk;
    if (world < 1 || world > 32 || T_local < 1 || H < 8 || H % 8 != 0 || top_k < 1 || top_k > 8 || bytes == nullptr) return MSK_ERR_INVALID;
    *bytes = ep_layout(world, T_local, H, top_k).total;
    return 0;
}

extern "C" int msk_ep_region_alloc(size_t bytes, void** ptr, void* handle64) {
    if (ptr == nullptr || handle64 == nullptr || bytes == 0) return MSK_ERR_INVALID;
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) return MSK_ERR_CUDA;
    if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
        cudaFree(p);
        return MSK_ERR_CUDA;
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
    if (cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle64), p) != cudaSuccess) {
        cudaFree(p);
        return MSK_ERR_CUDA;
    }
    *ptr = p;
    return 0;
}

extern "C" int msk_ep_region_open(const void* handle64, void** ptr) {
    if (ptr == nullptr || handle64 == nullptr) return MSK_ERR_INVALID;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof h);
    return cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? 0 : MSK_ERR_CUDA;
}

extern "C" int msk_ep_region_close(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? 0 : MSK_ERR_CUDA; }
extern "C" int msk_ep_region_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? 0 : MSK_ERR_CUDA; }

extern "C" int msk_selftest_flag_timeout(const int32_t* flag, long long wait_cycles, int* status, void* stream) {
    if (flag == nullptr || status == nullptr || wait_cycles < 1) return MSK_ERR_INVALID;
    msk::flag_timeout_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(flag, wait_cycles, status);
    return cudaGetLastError() == cudaSuccess ? 0 : MSK_ERR_CUDA;
}

extern "C" int msk_ep_step(const MskEpStep* q, int* status, void* stream) {
    using namespace msk;
    if (q == nullptr) return MSK_ERR_INVALID;
    const MskEpComm& c = q->comm;
    const MskLayerFront& f = q->front;
    const int T_local = f.B * f.L, H = f.H, k = f.top_k;
    if (c.world < 1 || c.world > 32 || c.rank < 0 || c.rank >= c.world || c.T_local != T_local || c.step < 1 || !c.self || !c.peers ||
        !c.counters || !q->out || c.n_experts % c.world != 0 || H > 8192)
        return MSK_ERR_INVALID;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const EpLayout lay = ep_layout(c.world, T_local, H, k);
    const int par = c.step & 1;
    const long long budget = c.wait_cycles > 0 ? c.wait_cycles : kWaitBudgetCycles;
    const size_t rows_off = lay.rows_off + static_cast<size_t>(par) * c.world * T_local * lay.row_bytes;
    const size_t recv_off = lay.recv_off + static_cast<size_t>(par) * c.world * T_local * H * sizeof(float);

    int rc = msk_layer_front(&f, status, stream);
    if (rc != 0) return rc;

    EpDispatchArgs d{};
    d.xn = static_cast<const uint16_t*>(f.xn1), d.ids = f.topk_ids, d.wts = f.topk_weights;
    d.ssq = f.ssq1 + static_cast<size_t>((H + 127) / 128) * T_local;  // the router's totals
    d.peers = c.peers, d.world = c.world, d.rank = c.rank, d.T_local = T_local, d.H = H, d.top_k = k;
    d.row_bytes = lay.row_bytes, d.step = c.step, d.rows_off = rows_off, d.flag_off = lay.dflag(par, c.rank);
    d.counter = c.counters;
    rc = launch_ep(ep_dispatch_kernel, T_local, s, d);
    if (rc != 0) return rc;

    char* self = static_cast<char*>(c.self);
    char* rows = self + rows_off;
    MskEpHooks hk{};
    hk.wait_flags = reinterpret_cast<const int32_t*>(self + lay.dflag(par, 0)), hk.wait_count = c.world, hk.wait_value = c.step;
    hk.wait_cycles = budget;
    hk.peers = c.peers, hk.n_peers = c.world, hk.rows_per_peer = T_local;
    hk.out_off = recv_off + static_cast<size_t>(c.rank) * T_local * H * sizeof(float);
    hk.flag_off = lay.cflag(par, c.rank), hk.flag_value = c.step, hk.done_counter = c.counters + 1;
    MskMoeParams m = q->moe;
    m.x = rows, m.ldx = lay.row_bytes / 2, m.x_fp16 = 1;
    m.topk_ids = reinterpret_cast<int32_t*>(rows + 2 * H), m.topk_weights = reinterpret_cast<float*>(rows + 2 * H + 4 * k);
    m.ld_topk = lay.row_bytes / 4, m.logits = nullptr, m.top_k = k;
    m.x_ssq = reinterpret_cast<const float*>(rows + lay.row_bytes - 16), m.x_ssq_parts = 1, m.x_ssq_tstride = lay.row_bytes / 4;
    m.x_inv_dim = 1.0f / H, m.x_eps = f.norm_eps;
    m.T = c.world * T_local, m.H = H;
    m.local_start = c.rank * (c.n_experts / c.world), m.local_count = c.n_experts / c.world;
    m.resid = nullptr, m.out = nullptr, m.out_fp32 = 1, m.ldo = H, m.out_copy = nullptr;
    m.pdl = 1, m.ep = &hk;
    rc = msk_moe_forward(&m, status, stream);
    if (rc != 0) return rc;

    EpReduceArgs r{};
    r.stream1 = f.stream1, r.ids = f.topk_ids, r.recv = reinterpret_cast<const float*>(self + recv_off);
    r.flags = reinterpret_cast<const int*>(self + lay.cflag(par, 0));
    r.world = c.world, r.T_local = T_local, r.H = H, r.top_k = k, r.experts_per_rank = c.n_experts / c.world, r.step = c.step;
    r.wait_cycles = budget, r.out = q->out, r.out_bf16 = static_cast<__nv_bfloat16*>(q->hidden), r.status = status;
    return launch_ep(ep_reduce_peer_kernel, T_local, s, r);
}

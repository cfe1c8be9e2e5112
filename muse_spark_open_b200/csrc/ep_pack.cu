// Kernels on either side of the expert-parallel token exchange.
//   ep_pack    (home rank, before dispatch) one row per local token: the un-normalised BF16 expert input,
//              its chosen experts and their weights, and its sum of squares, laid out so that the gathered
//              buffer can be handed to the expert GEMMs as it is (strided views, no unpack pass).
//   ep_reduce  (home rank, after combine) stream_out[t] = stream1[t] + sum over ranks of that rank's
//              weighted, post-normed expert partial for token t, added in rank order (reproducible),
//              plus a BF16 copy.
// Row layout in bytes: [0, 2H) x bf16 | 4k expert ids int32 | 4k weights fp32 | pad to 16 | ssq fp32 + 12 padding.
#include "msk.h"
#include "ptx.cuh"

namespace msk {

__global__ void __launch_bounds__(256) ep_pack_kernel(const __nv_bfloat16* __restrict__ xn, const int* __restrict__ ids,
                                                      const float* __restrict__ wts, const float* __restrict__ ssq,
                                                      int ssq_parts, uint8_t* __restrict__ rows, int T, int H, int top_k,
                                                      int row_bytes) {
    const int t = blockIdx.x, tid = threadIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    uint8_t* row = rows + static_cast<size_t>(t) * row_bytes;
    const uint4* src = reinterpret_cast<const uint4*>(xn + static_cast<size_t>(t) * H);
    for (int i = tid; i < H / 8; i += 256) reinterpret_cast<uint4*>(row)[i] = __ldcg(src + i);
    if (tid < top_k) {
        reinterpret_cast<int*>(row + 2 * H)[tid] = __ldcg(ids + t * top_k + tid);
        reinterpret_cast<float*>(row + 2 * H + 4 * top_k)[tid] = __ldcg(wts + t * top_k + tid);
    }
    if (tid == 32) {
        float s = 0.0f;
        for (int q = 0; q < ssq_parts; ++q) s += __ldcg(ssq + q * T + t);
        float* tail = reinterpret_cast<float*>(row + row_bytes - 16);
        tail[0] = s, tail[1] = 0.0f, tail[2] = 0.0f, tail[3] = 0.0f;
    }
}

__global__ void __launch_bounds__(256) ep_reduce_kernel(const float* __restrict__ stream1, const float* __restrict__ recv,
                                                        int ranks, float* __restrict__ out, __nv_bfloat16* __restrict__ out_bf16,
                                                        int T, int H) {
    const int t = blockIdx.x, tid = threadIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    for (int d = tid * 4; d < H; d += 1024) {
        float4 acc = __ldcg(reinterpret_cast<const float4*>(stream1 + static_cast<size_t>(t) * H + d));
        for (int r = 0; r < ranks; ++r) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(recv + (static_cast<size_t>(r) * T + t) * H + d));
            acc.x += v.x, acc.y += v.y, acc.z += v.z, acc.w += v.w;
        }
        *reinterpret_cast<float4*>(out + static_cast<size_t>(t) * H + d) = acc;
        if (out_bf16 != nullptr)
            *reinterpret_cast<uint2*>(out_bf16 + static_cast<size_t>(t) * H + d) =
                make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
    }
}

}  // namespace msk

extern "C" int msk_ep_row_bytes(int H, int top_k) { return 2 * H + ((8 * top_k + 15) & ~15) + 16; }

extern "C" int msk_ep_pack(const void* xn, const int32_t* topk_ids, const float* topk_weights, const float* ssq,
                           int ssq_parts, void* rows, int T, int H, int top_k, void* stream) {
    using namespace msk;
    if (!xn || !topk_ids || !topk_weights || !ssq || !rows || T < 1 || H % 8 != 0 || top_k < 1 || top_k > 32) return MSK_ERR_INVALID;
    ep_pack_kernel<<<T, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(xn), topk_ids,
                                                                      topk_weights, ssq, ssq_parts, static_cast<uint8_t*>(rows),
                                                                      T, H, top_k, msk_ep_row_bytes(H, top_k));
    return cudaGetLastError() == cudaSuccess ? 0 : MSK_ERR_CUDA;
}

extern "C" int msk_ep_reduce(const float* stream1, const float* recv, int ranks, float* out, void* out_bf16, int T, int H,
                             void* stream) {
    using namespace msk;
    if (!stream1 || !recv || !out || ranks < 1 || T < 1 || H % 4 != 0) return MSK_ERR_INVALID;
    ep_reduce_kernel<<<T, 256, 0, static_cast<cudaStream_t>(stream)>>>(stream1, recv, ranks, out,
                                                                        static_cast<__nv_bfloat16*>(out_bf16), T, H);
    return cudaGetLastError() == cudaSuccess ? 0 : MSK_ERR_CUDA;
}

// Layout self-tests: one 128-thread CTA computes one small product through each operand path the
// production kernels use, so that a wrong descriptor, swizzle or TMEM mapping shows up as a wrong
// number on a toy case rather than inside a large kernel.
//   mode 0  bf16, A and B K-major, both staged by 2-D TMA with the 128-byte swizzle   (projection)
//   mode 1  e4m3, A K-major from a paged cache by 4-D TMA, B K-major written by threads (scores)
//   mode 2  e4m3, A MN-major from a paged cache by 4-D TMA, B K-major written by threads (values)
//   mode 3  bf16, A written to tensor memory by tcgen05.st, B K-major by cp.async       (experts)
// (kind::f16 wants both operands in the same format: FP16 x BF16 in one MMA ends in a CUDA error.)
#include "msk.h"
#include "ptx.cuh"
#include "tmap.cuh"

namespace msk {

struct SelftestArgs {
    const void* a;
    const void* b;
    float* d;
    int n;
    int mode;
    int* status;
};

__global__ void __launch_bounds__(128) selftest_kernel(const __grid_constant__ CUtensorMap tm_a,
                                                       const __grid_constant__ CUtensorMap tm_b, SelftestArgs p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[2];
    __shared__ uint32_t tmem_slot;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t sa = base, sb = base + 16384;  // A tile (16 KB), then B tile
    const uint32_t bar_full = smem_u32(&bars[0]), bar_done = smem_u32(&bars[1]);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int where = (MSK_K_SELFTEST << 8) | p.mode;
    const int n = p.n;
    constexpr uint32_t kCols = 256;  // D in columns [0, 128), A (mode 3) in columns [128, 160)

    if (warp == 0) {
        tmem_alloc(smem_u32(&tmem_slot), kCols);
        tmem_relinquish();
    }
    if (tid == 0) {
        mbar_init(bar_full, 1);
        mbar_init(bar_done, 1);
        fence_mbar_init();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;

    // ---- stage operands
    if (p.mode == 0) {
        if (tid == 0) {
            mbar_expect_tx(bar_full, 16384 + n * 128);
            tma_load_2d(sa, &tm_a, bar_full, 0, 0);
            tma_load_2d(sb, &tm_b, bar_full, 0, 0);
        }
    } else if (p.mode == 1 || p.mode == 2) {
        if (tid == 0) {
            mbar_expect_tx(bar_full, 16384);
            tma_load_4d(sa, &tm_a, bar_full, 0, 0, 0, 1);          // keys 0..63 come from page 1
            tma_load_4d(sa + 8192, &tm_a, bar_full, 0, 0, 0, 0);   // keys 64..127 from page 0
        }
        // B[n][128 bytes] row-major in global -> swizzled K-major rows in shared memory
        const uint8_t* b = static_cast<const uint8_t*>(p.b);
        for (int i = tid; i < n * 8; i += 128) {
            const int row = i >> 3, chunk = i & 7;
            const uint4 v = *reinterpret_cast<const uint4*>(b + row * 128 + chunk * 16);
            *reinterpret_cast<uint4*>(gen + 16384 + swz128(row, chunk * 16)) = v;
        }
        fence_proxy_async_smem();
    } else {
        // A row `tid` (64 bf16 = 32 words) -> tensor memory lane tid, columns [128, 160)
        const uint32_t* a = static_cast<const uint32_t*>(p.a) + tid * 32;
        uint32_t r[16];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int j = 0; j < 16; ++j) r[j] = a[h * 16 + j];
            tmem_st16(tmem + (static_cast<uint32_t>(warp * 32) << 16) + 128 + h * 16, r);
        }
        tmem_wait_st();
        const uint8_t* b = static_cast<const uint8_t*>(p.b);
        for (int i = tid; i < n * 8; i += 128) {
            const int row = i >> 3, chunk = i & 7;
            cp_async_16(sb + swz128(row, chunk * 16), b + row * 128 + chunk * 16, 16);
        }
        asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
        fence_proxy_async_smem();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    // ---- one thread issues the MMAs
    if (warp == 0) {
        bool ok = true;
        if (p.mode != 3) ok = mbar_wait(bar_full, 0, p.status, where);
        tc_fence_after();
        if (lane == 0 && ok) {
            if (p.mode == 0 || p.mode == 3) {
                const uint32_t idesc = umma_idesc(128, n, 1, 1, 0, 0);
                const uint64_t bd = umma_smem_desc(sb, 16, 1024, kSwizzle128);
                const uint64_t ad = umma_smem_desc(sa, 16, 1024, kSwizzle128);
                for (int k = 0; k < 4; ++k) {  // K = 64 in steps of 16 elements = 32 bytes
                    if (p.mode == 0) umma_f16_ss(tmem, ad + 2 * k, bd + 2 * k, idesc, k != 0);
                    else umma_f16_ts(tmem, tmem + 128 + 8 * k, bd + 2 * k, idesc, k != 0);
                }
            } else if (p.mode == 1) {
                const uint32_t idesc = umma_idesc(128, n, 0, 0, 0, 0);
                const uint64_t ad = umma_smem_desc(sa, 16, 1024, kSwizzle128);
                const uint64_t bd = umma_smem_desc(sb, 16, 1024, kSwizzle128);
                for (int k = 0; k < 4; ++k) umma_f8_ss(tmem, ad + 2 * k, bd + 2 * k, idesc, k != 0);  // 32 B per step
            } else {
                const uint32_t idesc = umma_idesc(128, n, 0, 0, 1, 0);
                const uint64_t bd = umma_smem_desc(sb, 16, 1024, kSwizzle128);
                for (int k = 0; k < 4; ++k) {  // 32 keys = 32 rows of 128 B per step
                    const uint64_t ad = umma_smem_desc(sa + 4096 * k, 1024, 1024, kSwizzle128);
                    umma_f8_ss(tmem, ad, bd + 2 * k, idesc, k != 0);
                }
            }
            umma_commit(bar_done);
        }
        __syncwarp();
    }
    const bool done = mbar_wait(bar_done, 0, p.status, where);
    tc_fence_after();
    if (done) {
        for (int c = 0; c < n; c += 16) {
            uint32_t r[16];
            tmem_ld16(tmem + (static_cast<uint32_t>(warp * 32) << 16) + c, r);
            tmem_wait_ld();
            for (int j = 0; j < 16; ++j) p.d[tid * n + c + j] = __uint_as_float(r[j]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kCols);
}

}  // namespace msk

extern "C" int msk_selftest_umma(int mode, const void* a, const void* b, float* d, int n, int* status,
                                 void* stream) {
    using namespace msk;
    if (mode < 0 || mode > 3 || n < 16 || n > 128 || n % 16 != 0 || !a || !b || !d) return MSK_ERR_INVALID;
    CUtensorMap tm_a, tm_b;
    int rc = 0;
    if (mode == 0) {
        rc = make_tmap_bf16_2d(&tm_a, a, 128, 64, 64, 128);
        if (rc == 0) rc = make_tmap_bf16_2d(&tm_b, b, n, 64, 64, n);
    } else if (mode == 1 || mode == 2) {
        // cache [2 pages][64 tokens][1 head][128 bytes]
        const uint64_t dims[4] = {128, 1, 64, 2};
        const uint64_t strides[3] = {128, 128, 64 * 128};
        const uint32_t box[4] = {128, 1, 64, 1};
        rc = make_tmap(&tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        tm_b = tm_a;
    } else {
        rc = make_tmap_bf16_2d(&tm_a, b, n, 64, 64, 16);  // unused by the kernel; keeps the params valid
        tm_b = tm_a;
    }
    if (rc != 0) return rc;
    const int smem = 1024 + 16384 + 256 * 128;
    cudaError_t e = cudaFuncSetAttribute(selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return MSK_ERR_CUDA;
    SelftestArgs args{a, b, d, n, mode, status};
    selftest_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(tm_a, tm_b, args);
    return cudaGetLastError() == cudaSuccess ? 0 : MSK_ERR_CUDA;
}

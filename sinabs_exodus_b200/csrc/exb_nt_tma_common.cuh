// [N,T] layout through TMA: what the forward (exb_lif_nt_tma.cuh) and backward (exb_tma_lif_nt_bwd.cu) kernels
// share.  Include after exb_tma_common.cuh.
//
// Row classes.  A TMA box row should be one whole 128-byte line of global memory, or every piece ends in partial
// sectors.  Row n of an [N,T] tensor starts n*T floats into it, so its position inside a line repeats with period
// p = 32 / gcd(T mod 32, 32) rows (p <= 8 when T % 4 == 0).  The tensor is therefore described to TMA as
// [N/p][p][T], and a CTA owns 128 rows of ONE class j (rows j, j+p, j+2p, ...): they all start at the same position
// a_j inside their lines, and a box of [32 steps x 1 class x 32 rows] placed at time coordinate 32k - a_j consists of
// whole lines.  A load may start at a negative time coordinate (the fill is ignored), a store may not: the chunk
// that holds a class's first steps is stored by the warps themselves when a_j > 0.
#pragma once

namespace exb {

constexpr int NTT_WARPS = 4;               // consumer warps per CTA
constexpr int NTT_ROWS = NTT_WARPS * 32;   // rows per CTA (one thread per row)
constexpr int NTT_BOX_T = 32;              // time steps per box (128 bytes: the swizzle span)
constexpr int NTT_STAGE = NTT_ROWS * NTT_BOX_T;   // floats of one stage: 128 rows x 32 steps (16 KB)


__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, int x, int y, int z, uint32_t src)
{
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(src)
                 : "memory");
}

__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all stores of this thread's groups have finished READING shared memory (the data may still be on its way to DRAM)
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// makes this thread's shared-memory writes visible to the async (TMA) proxy
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Number of row classes of an [N,T] tensor , as log2; -1 when rows do not start on 16-byte boundaries.
static int nt_class_log2(int64_t T)
{
    if (T % 4) return -1;
    const int tm = (int)(T & 31);
    if (tm == 0) return 0;
    if (tm % 16 == 0) return 1;
    if (tm % 8 == 0) return 2;
    return 3;
}

// 3-D map of an [N,T] tensor seen as [N/p][p][T]: x = time (contiguous), y = class, z = row of the class;
// boxes of [32 x 1 x 32] with the 128-byte swizzle.
static bool make_nt_tensor_map(CUtensorMap *map, const float *base, int64_t N, int64_t T, int lp)
{
    PFN_cuTensorMapEncodeTiled enc = get_encode_fn();
    if (!enc || !base) return false;
    const int64_t p = 1ll << lp;
    if ((reinterpret_cast<uintptr_t>(base) & 15u) || (T % 4) || T < 64 || N <= 0 || (N % p)) return false;
    if (T > (1ll << 31) - 64 || N > (1ll << 31) - NTT_ROWS) return false;
    cuuint64_t gdim[3] = {(cuuint64_t)T, (cuuint64_t)p, (cuuint64_t)(N / p)};
    cuuint64_t gstr[2] = {(cuuint64_t)T * 4u, (cuuint64_t)(T * p) * 4u};
    cuuint32_t box[3] = {(cuuint32_t)NTT_BOX_T, 1u, 32u};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float *>(base), gdim, gstr, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

}  // namespace exb

// Single-tile tcgen05 GEMM through the same TMA tiles, shared-memory descriptors and TMEM read-out as the scan
// kernels, for every operand orientation they use.  D[128, N] = op(A) * op(B), bf16 in, fp32 out.
//   mode bit 0: A is MN-major (A given as [K, 128], the M axis contiguous)     else K-major (A given as [128, K])
//   mode bit 1: B is MN-major (B given as [K, N],  the N axis contiguous)      else K-major (B given as [N, K])
//   mode bit 2: A reaches shared memory through registers (manual 128-byte swizzle) instead of TMA (K-major only)
//   mode bit 3: A is staged in TMEM (packed bf16 pairs written with tcgen05.st) instead of shared memory (K-major only)
#include "common.cuh"
#include "tc_common.cuh"
#include "../../include/orbit_b200.h"

namespace orbit {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || p == nullptr) return nullptr;
  fn = (EncodeTiledFn)p;
  return fn;
}

static int make_tensor_map(CUtensorMap* out, CUtensorMapDataType dt, const void* base, int rank, const uint64_t* dims,
                           const uint64_t* strides_bytes, const uint32_t* box) {
  EncodeTiledFn enc = get_encode();
  ORBIT_REQUIRE(enc != nullptr, ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  ORBIT_REQUIRE(rank >= 1 && rank <= 5, ERR_BAD_ARG, "tensor map rank %d", rank);
  ORBIT_REQUIRE(aligned16(base), ERR_UNSUPPORTED, "tensor map base address must be 16-byte aligned");
  cuuint64_t gd[5], gs[5];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) {
    gd[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i > 0) {
      ORBIT_REQUIRE(strides_bytes[i - 1] % 16 == 0, ERR_UNSUPPORTED, "tensor map stride %llu bytes is not a multiple of 16",
                    (unsigned long long)strides_bytes[i - 1]);
      gs[i - 1] = strides_bytes[i - 1];
    }
  }
  CUresult r = enc(out, dt, (cuuint32_t)rank, const_cast<void*>(base), gd, gs, bx, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  ORBIT_REQUIRE(r == CUDA_SUCCESS, ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return OK;
}

int make_tensor_map_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                         const uint32_t* box) {
  return make_tensor_map(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, base, rank, dims, strides_bytes, box);
}
int make_tensor_map_f32(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                        const uint32_t* box) {
  return make_tensor_map(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, base, rank, dims, strides_bytes, box);
}

__global__ void __launch_bounds__(128) umma_selftest_kernel(const __grid_constant__ CUtensorMap tmA,
                                                            const __grid_constant__ CUtensorMap tmB,
                                                            const __nv_bfloat16* __restrict__ Ag, float* __restrict__ D,
                                                            int mode, int K, int N, int* __restrict__ status) {
  using namespace tc;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;               // 32 KB
  uint8_t* sB = smem + 32768;       // 32 KB
  __shared__ uint64_t bar_load, bar_mma;
  __shared__ uint32_t tmem_slot;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool a_mn = mode & 1, b_mn = mode & 2, a_manual = mode & 4, a_tmem = mode & 8;

  if (tid == 0) {
    mbar_init(&bar_load, 1);
    mbar_init(&bar_mma, 1);
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 256);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = tmem_slot;
  const uint32_t TM_A = 128;             // A operand in TMEM: K / 2 columns
  bool ok = true;

  if (tid == 0) {
    uint32_t bytes = 0;
    if (!a_manual && !a_tmem) bytes += 128 * K * 2;
    bytes += N * K * 2;
    mbar_expect_tx(&bar_load, bytes);
    if (!a_manual && !a_tmem) {
      if (!a_mn) for (int kb = 0; kb < K / 64; ++kb) tma_load_2d(sA + kb * 16384, &tmA, &bar_load, kb * 64, 0);
      else for (int mb = 0; mb < 2; ++mb) tma_load_2d(sA + mb * (K * 128), &tmA, &bar_load, mb * 64, 0);
    }
    if (!b_mn) for (int kb = 0; kb < K / 64; ++kb) tma_load_2d(sB + kb * (N * 128), &tmB, &bar_load, kb * 64, 0);
    else for (int nb = 0; nb < N / 64; ++nb) tma_load_2d(sB + nb * (K * 128), &tmB, &bar_load, nb * 64, 0);
  }
  if (a_manual) {
    // thread = row; 16-byte chunks of the row go to their swizzled place
    for (int c = 0; c < K / 8; ++c) {
      uint4 v = *reinterpret_cast<const uint4*>(Ag + (size_t)tid * K + c * 8);
      *reinterpret_cast<uint4*>(sA + (c / 8) * 16384 + sw128_offset(tid, c % 8)) = v;
    }
    fence_proxy_async();
  }
  if (a_tmem) {
    // thread = row = TMEM lane; 32 bf16 (16 packed columns) per store
    for (int c0 = 0; c0 < K / 32; ++c0) {
      uint32_t r[16];
      const uint4* src = reinterpret_cast<const uint4*>(Ag + (size_t)tid * K + c0 * 32);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint4 v = src[j];
        r[4 * j] = v.x; r[4 * j + 1] = v.y; r[4 * j + 2] = v.z; r[4 * j + 3] = v.w;
      }
      tmem_st16(tmem_addr(tbase, warp * 32, TM_A + c0 * 16), r);
    }
    tmem_st_wait();
    tc_fence_before_sync();
  }
  __syncthreads();
  if (!mbar_wait(&bar_load, 0)) ok = false;
  tc_fence_after_sync();
  if (tid == 0 && ok) {
    const uint32_t idesc = idesc_bf16(128, N, a_mn ? 1 : 0, b_mn ? 1 : 0);
    const uint32_t a0 = smem_u32(sA), b0 = smem_u32(sB);
    for (int ks = 0; ks < K / 16; ++ks) {
      uint64_t ad = a_mn ? smem_desc_sw128(a0 + ks * 2048, K * 128, 1024)
                         : smem_desc_sw128(a0 + (ks / 4) * 16384 + (ks % 4) * 32, 16, 1024);
      uint64_t bd = b_mn ? smem_desc_sw128(b0 + ks * 2048, K * 128, 1024)
                         : smem_desc_sw128(b0 + (ks / 4) * (N * 128) + (ks % 4) * 32, 16, 1024);
      if (a_tmem) umma_bf16_ta(tbase, tbase + TM_A + ks * 8, bd, idesc, ks > 0 ? 1u : 0u);
      else umma_bf16(tbase, ad, bd, idesc, ks > 0 ? 1u : 0u);
    }
    umma_commit(&bar_mma);
  }
  __syncwarp();
  if (ok && !mbar_wait(&bar_mma, 0)) ok = false;
  tc_fence_after_sync();
  if (ok) {
    for (int c0 = 0; c0 < N; c0 += 32) {
      uint32_t r[32];
      tmem_ld32(tmem_addr(tbase, warp * 32, c0), r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) D[(size_t)(warp * 32 + lane) * N + c0 + j] = __uint_as_float(r[j]);
    }
  } else if (lane == 0) {
    atomicExch(status, 1);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 256);
}

// The wind-down every tensor-core kernel of this library performs when a bounded wait runs out, by itself: the CTA
// holds TMEM and waits (at most `polls` polls) on an mbarrier that nothing arrives on; the wait gives up, the status
// word is set, TMEM is freed and the kernel returns normally.
__global__ void __launch_bounds__(128) wait_timeout_selftest_kernel(int* __restrict__ status, uint32_t polls) {
  using namespace tc;
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 32);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = tmem_slot;
  const bool done = mbar_wait(&bar, 0, polls);
  if (!done && tid == 0) atomicExch(status, 1);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 32);
}

}  // namespace orbit

using namespace orbit;

extern "C" int orbit_selftest_wait_timeout(int* status, int polls, void* stream) {
  ORBIT_REQUIRE(status != nullptr, ERR_BAD_ARG, "orbit_selftest_wait_timeout: null status pointer");
  ORBIT_REQUIRE(polls >= 1 && polls <= 4096, ERR_UNSUPPORTED, "orbit_selftest_wait_timeout: polls must be in [1, 4096], got %d", polls);
  wait_timeout_selftest_kernel<<<1, 128, 0, (cudaStream_t)stream>>>(status, (uint32_t)polls);
  ORBIT_CHECK_LAUNCH("wait_timeout_selftest_kernel");
  return OK;
}

extern "C" int orbit_selftest_umma(const void* A, const void* B, float* D, int mode, int K, int N, int* status,
                                   void* stream) {
  ORBIT_REQUIRE(A && B && D && status, ERR_BAD_ARG, "orbit_selftest_umma: null pointer");
  ORBIT_REQUIRE((K == 64 || K == 128) && (N == 64 || N == 128) && mode >= 0 && mode < 16 && !((mode & 12) && (mode & 1)) &&
                    (mode & 12) != 12,
                ERR_UNSUPPORTED, "orbit_selftest_umma: K, N in {64, 128}; A through registers or TMEM is K-major only");
  CUtensorMap tmA, tmB;
  int rc;
  {
    uint64_t dims[2], str[1];
    uint32_t box[2];
    if (mode & 1) { dims[0] = 128; dims[1] = K; str[0] = 128 * 2; box[0] = 64; box[1] = K; }
    else { dims[0] = K; dims[1] = 128; str[0] = (uint64_t)K * 2; box[0] = 64; box[1] = 128; }
    if ((rc = make_tensor_map_bf16(&tmA, A, 2, dims, str, box)) != OK) return rc;
    if (mode & 2) { dims[0] = N; dims[1] = K; str[0] = (uint64_t)N * 2; box[0] = 64; box[1] = K; }
    else { dims[0] = K; dims[1] = N; str[0] = (uint64_t)K * 2; box[0] = 64; box[1] = N; }
    if ((rc = make_tensor_map_bf16(&tmB, B, 2, dims, str, box)) != OK) return rc;
  }
  const int smem = 65536 + 1024;
  ORBIT_CHECK_CUDA(cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  umma_selftest_kernel<<<1, 128, smem, (cudaStream_t)stream>>>(tmA, tmB, (const __nv_bfloat16*)A, D, mode, K, N, status);
  ORBIT_CHECK_LAUNCH("umma_selftest_kernel");
  return OK;
}

// SSD-MIMO chunked scan, precision "io": bf16 operands on tcgen05 tensor cores (fp32 accumulators in TMEM, fp32
// clocks/decays/states), tiles fed by TMA.  Envelope of this file: SISO kernel heads (R = O = 1), N = 128 state rows,
// G = 64 channels per head, head-shared maps (no gates, no per-head biases, no sibling mix), chunk T = 128.
//
// One CTA owns one (batch, chunk) and loops over heads.  Tiles in shared memory are [rows x 64 bf16] blocks with the
// 128-byte swizzle (what TMA writes); one buffer serves both a K-major and an MN-major tcgen05 descriptor:
//   map tile  B|C [128 tokens][128 n]  = two 64-column blocks, 16 KB apart
//   drive     u|dy [128 tokens][64 p]  = one block
// Contractions per head (M = 128 always):
//   chunk_state / chunk_dstate :  Z[n,p]  = sum_s map[s,n] * (f_s x[s,p])            A: map MN-major, B: scaled x MN-major
//   chunk_out                  :  Y1[t,p] = sum_s (CB o W)[t,s] u[s,p]               A: mask K-major (through registers), B: u MN-major
//                                 Y2[t,p] = sum_n C[t,n] Sin[n,p]                    A: C K-major, B: Sin MN-major
//   with CB[t,s] = sum_n C[t,n] B[s,n] once per CTA (shared by every head).
#include "common.cuh"
#include "scan_args.h"
#include "tc_common.cuh"

namespace orbit {
using namespace tc;

constexpr int TC_T = 128, TC_N = 128, TC_G = 64, TC_THREADS = 256;
constexpr uint32_t BLK = 128 * 128;   // bytes of one [128 x 64] bf16 block

// ---- bounded waits with a CTA-wide abort flag --------------------------------------------------------------------
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  uint32_t addr = smem_u32(bar);
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((i & 63u) == 63u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

// Inclusive prefix over the 128 values held by threads 0..127 -> cs[0..127]; every thread of the CTA must call.
__device__ __forceinline__ void chunk_prefix(float v, float* cs, float* wsum) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float x = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    float y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  if (warp < 4 && lane == 31) wsum[warp] = x;
  __syncthreads();
  if (warp < 4) {
    float off = 0.f;
    for (int w = 0; w < warp; ++w) off += wsum[w];
    cs[tid] = x + off;
  }
  __syncthreads();
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void unpack_bf16(uint32_t w, float& lo, float& hi) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&w);
  lo = __low2float(v);
  hi = __high2float(v);
}

__device__ __forceinline__ uint8_t* align1024(uint8_t* p) { return (uint8_t*)(((uintptr_t)p + 1023) & ~(uintptr_t)1023); }

// K-major descriptor of k-step `ks` (16 columns) of a [128 x 128] operand stored as two 64-column blocks
__device__ __forceinline__ uint64_t desc_k(uint32_t base, int ks) {
  return smem_desc_sw128(base + (uint32_t)(ks >> 2) * BLK + (uint32_t)(ks & 3) * 32u, 16u, 1024u);
}
// MN-major descriptor of k-step `ks` (16 rows); 64-wide MN blocks are BLK bytes apart
__device__ __forceinline__ uint64_t desc_mn(uint32_t base, int ks) { return smem_desc_sw128(base + (uint32_t)ks * 2048u, BLK, 1024u); }

// ------------------------------------------------------------------------------------------------------------------
// chunk_state (mode 0):  Z[n,p] = sum_s B[s,n] e_s u[s,p],   e_s = exp(cs_T - cs_s) w_s          -> a.Sin, a.atot
// chunk_dstate (mode 1): Gs[n,p] = sum_t C[t,n] a_t dy[t,p], a_t = exp(cs_t)                      -> a.dS
// ------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(TC_THREADS, 1) tc_chunk_state_kernel(const __grid_constant__ CUtensorMap tmM,
                                                                       const __grid_constant__ CUtensorMap tmX,
                                                                       const ScanArgs a, const int mode) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = align1024(smem_raw);
  uint8_t* sM = sm;                      // map tile, 2 blocks
  uint8_t* sX = sm + 2 * BLK;            // raw drive tiles, 2 buffers
  uint8_t* sXs = sm + 4 * BLK;           // scaled drive tiles, 2 buffers
  float* cs = reinterpret_cast<float*>(sm + 6 * BLK);
  float* fv = cs + 128;
  float* wsum = fv + 128;
  __shared__ uint64_t bar_map, bar_x[2], bar_mma[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, q = warp & 3, wg = warp >> 2;
  const int c = blockIdx.x, b = blockIdx.y, t0 = c * TC_T;
  const int Tv = min(TC_T, a.L - t0);
  const int H = a.H;

  if (tid == 0) {
    mbar_init(&bar_map, 1);
    mbar_init(&bar_x[0], 1);
    mbar_init(&bar_x[1], 1);
    mbar_init(&bar_mma[0], 1);
    mbar_init(&bar_mma[1], 1);
    mbar_fence_init();
    s_abort = 0;
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 128);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = tmem_slot;
  volatile int* abort_flag = &s_abort;

  if (tid == 0) {
    mbar_expect_tx(&bar_map, 2 * BLK);
    tma_load_3d(sM, &tmM, &bar_map, 0, t0, b);
    tma_load_3d(sM + BLK, &tmM, &bar_map, 64, t0, b);
    for (int i = 0; i < 2 && i < H; ++i) {
      mbar_expect_tx(&bar_x[i], BLK);
      tma_load_3d(sX + i * BLK, &tmX, &bar_x[i], i * TC_G, t0, b);
    }
  }
  float* outbuf = mode == 0 ? a.Sin : a.dS;
  const uint32_t idesc = idesc_bf16(128, 64, 1, 1);

  auto epilogue = [&](int hh) {
    const int be = hh & 1;
    if (wait_or_abort(&bar_mma[be], (uint32_t)((hh >> 1) & 1), abort_flag)) {
      tc_fence_after_sync();
      uint32_t r[32];
      tmem_ld32(tmem_addr(tbase, q * 32, be * 64 + wg * 32), r);
      tmem_ld_wait();
      float* dst = outbuf + ((((int64_t)b * a.nc + c) * H + hh) * TC_N + (q * 32 + lane)) * (int64_t)TC_G + wg * 32;
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        *reinterpret_cast<float4*>(dst + j) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                          __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
    }
    tc_fence_before_sync();
  };

  for (int h = 0; h < H; ++h) {
    const int buf = h & 1;
    float d = 0.f, wt = 0.f;
    if (tid < Tv) {
      int64_t i = ((int64_t)b * a.L + t0 + tid) * H + h;
      d = a.dA[i];
      wt = a.w[i];
    }
    chunk_prefix(d, cs, wsum);
    if (tid < 128) fv[tid] = mode == 0 ? __expf(cs[127] - cs[tid]) * wt : __expf(cs[tid]);
    if (tid == 0 && mode == 0) a.atot[((int64_t)b * a.nc + c) * H + h] = __expf(cs[127]);
    __syncthreads();
    if (wait_or_abort(&bar_x[buf], (uint32_t)((h >> 1) & 1), abort_flag)) {
      const int row = tid & 127, half = tid >> 7;
      const float f = fv[row];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t off = buf * BLK + sw128_offset(row, half * 4 + j);
        uint4 v = *reinterpret_cast<const uint4*>(sX + off);
        uint32_t* pv = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float lo, hi;
          unpack_bf16(pv[k], lo, hi);
          pv[k] = pack_bf16(lo * f, hi * f);
        }
        *reinterpret_cast<uint4*>(sXs + off) = v;
      }
    }
    fence_proxy_async();
    __syncthreads();
    if (tid == 0 && !*abort_flag) {
      if (h + 2 < H) {
        mbar_expect_tx(&bar_x[buf], BLK);
        tma_load_3d(sX + buf * BLK, &tmX, &bar_x[buf], (h + 2) * TC_G, t0, b);
      }
      bool ok = (h > 0) || wait_or_abort(&bar_map, 0, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        const uint32_t am = smem_u32(sM), bx = smem_u32(sXs + buf * BLK);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) umma_bf16(tbase + buf * 64, desc_mn(am, ks), desc_mn(bx, ks), idesc, ks > 0 ? 1u : 0u);
        umma_commit(&bar_mma[buf]);
      }
    }
    if (h > 0) epilogue(h - 1);
  }
  epilogue(H - 1);
  __syncthreads();
  if (tid == 0 && *abort_flag && a.status) atomicExch(a.status, 1);
  if (warp == 0) tmem_dealloc(tbase, 128);
}

// ------------------------------------------------------------------------------------------------------------------
// chunk_out:  y[t,p] = sum_{s<=t} CB[t,s] W_h[t,s] u[s,p] + a_t sum_n C[t,n] Sin_h[n,p] + D[h,p] u[t,p]
// ------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(TC_THREADS, 1) tc_chunk_out_kernel(const __grid_constant__ CUtensorMap tmB,
                                                                     const __grid_constant__ CUtensorMap tmC,
                                                                     const __grid_constant__ CUtensorMap tmU,
                                                                     const ScanArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = align1024(smem_raw);
  uint8_t* sB = sm;                      // 2 blocks
  uint8_t* sC = sm + 2 * BLK;            // 2 blocks
  uint8_t* sX = sm + 4 * BLK;            // 2 buffers
  uint8_t* sMs = sm + 6 * BLK;           // masked scores [128 t][128 s], 2 blocks
  uint8_t* sS = sm + 8 * BLK;            // entering state [128 n][64 p] bf16, 1 block
  float* cs = reinterpret_cast<float*>(sm + 9 * BLK);
  float* wv = cs + 128;
  float* wdv = wv + 128;
  float* wsum = wdv + 128;
  __shared__ uint64_t bar_map, bar_x[2], bar_cb, bar_y;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, q = warp & 3, wg = warp >> 2;
  const int c = blockIdx.x, b = blockIdx.y, t0 = c * TC_T;
  const int Tv = min(TC_T, a.L - t0);
  const int H = a.H;
  const int t = q * 32 + lane;           // this thread's token row in TMEM

  if (tid == 0) {
    mbar_init(&bar_map, 1);
    mbar_init(&bar_x[0], 1);
    mbar_init(&bar_x[1], 1);
    mbar_init(&bar_cb, 1);
    mbar_init(&bar_y, 1);
    mbar_fence_init();
    s_abort = 0;
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 256);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = tmem_slot;
  volatile int* abort_flag = &s_abort;
  const uint32_t TM_CB = 0, TM_Y1 = 128, TM_Y2 = 192;

  if (tid == 0) {
    mbar_expect_tx(&bar_map, 4 * BLK);
    tma_load_3d(sB, &tmB, &bar_map, 0, t0, b);
    tma_load_3d(sB + BLK, &tmB, &bar_map, 64, t0, b);
    tma_load_3d(sC, &tmC, &bar_map, 0, t0, b);
    tma_load_3d(sC + BLK, &tmC, &bar_map, 64, t0, b);
    for (int i = 0; i < 2 && i < H; ++i) {
      mbar_expect_tx(&bar_x[i], BLK);
      tma_load_3d(sX + i * BLK, &tmU, &bar_x[i], i * TC_G, t0, b);
    }
    if (wait_or_abort(&bar_map, 0, abort_flag)) {
      tc_fence_after_sync();
      const uint32_t ac = smem_u32(sC), bb = smem_u32(sB);
      const uint32_t id = idesc_bf16(128, 128, 0, 0);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) umma_bf16(tbase + TM_CB, desc_k(ac, ks), desc_k(bb, ks), id, ks > 0 ? 1u : 0u);
      umma_commit(&bar_cb);
    }
  }
  __syncthreads();
  bool cb_ok = wait_or_abort(&bar_cb, 0, abort_flag);
  tc_fence_after_sync();
  const uint32_t idesc_y = idesc_bf16(128, 64, 0, 1);
  __nv_bfloat16* yout = reinterpret_cast<__nv_bfloat16*>(a.y);

  for (int h = 0; h < H; ++h) {
    const int buf = h & 1;
    float d = 0.f, wt = 0.f, wdt = 0.f;
    if (tid < Tv) {
      int64_t i = ((int64_t)b * a.L + t0 + tid) * H + h;
      d = a.dA[i];
      wt = a.w[i];
      wdt = a.wd[i];
    }
    if (tid < 128) {
      wv[tid] = wt;
      wdv[tid] = wdt;
    }
    chunk_prefix(d, cs, wsum);
    // entering state fp32 [n][p] -> bf16 swizzled rows (coalesced 16-byte loads)
    {
      const float4* src = reinterpret_cast<const float4*>(a.Sin + (((int64_t)b * a.nc + c) * H + h) * (int64_t)(TC_N * TC_G));
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int idx = it * TC_THREADS + tid;
        const int n = idx >> 4, c4 = idx & 15;
        float4 v = src[idx];
        uint2 pk = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
        *reinterpret_cast<uint2*>(sS + sw128_offset(n, c4 >> 1) + (c4 & 1) * 8) = pk;
      }
    }
    // masked scores: this thread owns row t, column slabs 2*wg and 2*wg+1 (32 columns each)
    if (cb_ok) {
      const float cst = cs[t], wdt_t = wdv[t];
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        const int j = wg * 2 + jj;
        uint32_t pk[16];
        if (j > q) {   // the whole warp sits above the diagonal for this slab
#pragma unroll
          for (int k = 0; k < 16; ++k) pk[k] = 0u;
        } else {
          uint32_t r[32];
          tmem_ld32(tmem_addr(tbase, q * 32, TM_CB + j * 32), r);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int s = j * 32 + i;
            float wgt = 0.f;
            if (s < t) wgt = __expf(cst - cs[s]) * wv[s];
            else if (s == t) wgt = wdt_t;
            v[i] = __uint_as_float(r[i]) * wgt;
          }
#pragma unroll
          for (int k = 0; k < 16; ++k) pk[k] = pack_bf16(v[2 * k], v[2 * k + 1]);
        }
        uint8_t* dstb = sMs + (j >> 1) * BLK;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          *reinterpret_cast<uint4*>(dstb + sw128_offset(t, (j & 1) * 4 + k)) = make_uint4(pk[4 * k], pk[4 * k + 1], pk[4 * k + 2], pk[4 * k + 3]);
      }
    }
    tc_fence_before_sync();
    fence_proxy_async();
    __syncthreads();
    if (tid == 0 && !*abort_flag) {
      if (wait_or_abort(&bar_x[buf], (uint32_t)((h >> 1) & 1), abort_flag)) {
        tc_fence_after_sync();
        const uint32_t am = smem_u32(sMs), bx = smem_u32(sX + buf * BLK), ac = smem_u32(sC), bs = smem_u32(sS);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) umma_bf16(tbase + TM_Y1, desc_k(am, ks), desc_mn(bx, ks), idesc_y, ks > 0 ? 1u : 0u);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) umma_bf16(tbase + TM_Y2, desc_k(ac, ks), desc_mn(bs, ks), idesc_y, ks > 0 ? 1u : 0u);
        umma_commit(&bar_y);
      }
    }
    if (wait_or_abort(&bar_y, (uint32_t)(h & 1), abort_flag)) {
      tc_fence_after_sync();
      uint32_t r1[32], r2[32];
      tmem_ld32(tmem_addr(tbase, q * 32, TM_Y1 + wg * 32), r1);
      tmem_ld32(tmem_addr(tbase, q * 32, TM_Y2 + wg * 32), r2);
      tmem_ld_wait();
      const float at = __expf(cs[t]);
      uint32_t outp[16];
#pragma unroll
      for (int k4 = 0; k4 < 4; ++k4) {
        uint4 uv = *reinterpret_cast<const uint4*>(sX + buf * BLK + sw128_offset(t, wg * 4 + k4));
        const uint32_t* up = reinterpret_cast<const uint32_t*>(&uv);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int i = k4 * 8 + k * 2;
          float u0, u1;
          unpack_bf16(up[k], u0, u1);
          float d0 = 0.f, d1 = 0.f;
          if (a.Dg) {
            d0 = a.Dg[h * TC_G + wg * 32 + i];
            d1 = a.Dg[h * TC_G + wg * 32 + i + 1];
          }
          float y0 = __uint_as_float(r1[i]) + at * __uint_as_float(r2[i]) + d0 * u0;
          float y1 = __uint_as_float(r1[i + 1]) + at * __uint_as_float(r2[i + 1]) + d1 * u1;
          outp[k4 * 4 + k] = pack_bf16(y0, y1);
        }
      }
      if (t < Tv) {
        uint4* dst = reinterpret_cast<uint4*>(yout + ((int64_t)b * a.L + t0 + t) * (int64_t)(H * TC_G) + h * TC_G + wg * 32);
#pragma unroll
        for (int k = 0; k < 4; ++k) dst[k] = make_uint4(outp[4 * k], outp[4 * k + 1], outp[4 * k + 2], outp[4 * k + 3]);
      }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (tid == 0 && !*abort_flag && h + 2 < H) {
      mbar_expect_tx(&bar_x[buf], BLK);
      tma_load_3d(sX + buf * BLK, &tmU, &bar_x[buf], (h + 2) * TC_G, t0, b);
    }
  }
  __syncthreads();
  if (tid == 0 && *abort_flag && a.status) atomicExch(a.status, 1);
  if (warp == 0) tmem_dealloc(tbase, 256);
}

// ------------------------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------------------------
int tc_supported(const ScanArgs& a, int dtype, const char** why) {
  *why = nullptr;
  if (dtype != BF16) *why = "activations must be bfloat16";
  else if (a.R != 1 || a.O != 1 || a.N != TC_N || a.G != TC_G) *why = "tensor-core tiles serve R = O = 1, N = 128, G = 64";
  else if (a.gBp || a.gCp || a.beta || a.gamma || a.chi) *why = "tensor-core tiles serve head-shared maps (no gates, per-head biases or sibling mix)";
  else if (a.T != TC_T) *why = "tensor-core tiles use chunk length 128";
  else if (a.b_ts % 8 || a.c_ts % 8 || !aligned16(a.Bhat) || !aligned16(a.Chat) || !aligned16(a.u)) *why = "maps and drive must be 16-byte aligned with token strides that are multiples of 8 elements";
  return *why == nullptr;
}

int tc_pick_chunk(int R, int O, int G, int N, int backward, int limit) {
  if (backward) return 0;   // backward tiles not built yet: training takes the fp32 kernels
  return (R == 1 && O == 1 && G == TC_G && N == TC_N && limit >= TC_T) ? TC_T : 0;
}

static int map_rows(CUtensorMap* m, const void* base, int cols, int64_t token_stride, int L, int B) {
  uint64_t dims[3] = {(uint64_t)cols, (uint64_t)L, (uint64_t)B};
  uint64_t str[2] = {(uint64_t)token_stride * 2, (uint64_t)token_stride * 2 * (uint64_t)L};
  uint32_t box[3] = {64, 128, 1};
  return make_tensor_map_bf16(m, base, 3, dims, str, box);
}

constexpr int SMEM_STATE = 6 * BLK + 2048 + 1024;
constexpr int SMEM_OUT = 9 * BLK + 2048 + 1024;

static int launch_state(const ScanArgs& a, int mode, cudaStream_t st) {
  CUtensorMap tmM, tmX;
  int rc;
  if (mode == 0) {
    if ((rc = map_rows(&tmM, a.Bhat, TC_N, a.b_ts, a.L, a.B)) != OK) return rc;
    if ((rc = map_rows(&tmX, a.u, a.H * TC_G, (int64_t)a.H * TC_G, a.L, a.B)) != OK) return rc;
  } else {
    ORBIT_REQUIRE(aligned16(a.dy), ERR_UNSUPPORTED, "dy must be 16-byte aligned");
    if ((rc = map_rows(&tmM, a.Chat, TC_N, a.c_ts, a.L, a.B)) != OK) return rc;
    if ((rc = map_rows(&tmX, a.dy, a.H * TC_G, (int64_t)a.H * TC_G, a.L, a.B)) != OK) return rc;
  }
  ORBIT_CHECK_CUDA(cudaFuncSetAttribute(tc_chunk_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_STATE));
  tc_chunk_state_kernel<<<dim3(a.nc, a.B), TC_THREADS, SMEM_STATE, st>>>(tmM, tmX, a, mode);
  ORBIT_CHECK_LAUNCH("tc_chunk_state_kernel");
  return OK;
}

int tc_launch_chunk_state(const ScanArgs& a, cudaStream_t st) { return launch_state(a, 0, st); }
int tc_launch_chunk_dstate(const ScanArgs& a, cudaStream_t st) { return launch_state(a, 1, st); }

int tc_launch_chunk_out(const ScanArgs& a, cudaStream_t st) {
  CUtensorMap tmB, tmC, tmU;
  int rc;
  if ((rc = map_rows(&tmB, a.Bhat, TC_N, a.b_ts, a.L, a.B)) != OK) return rc;
  if ((rc = map_rows(&tmC, a.Chat, TC_N, a.c_ts, a.L, a.B)) != OK) return rc;
  if ((rc = map_rows(&tmU, a.u, a.H * TC_G, (int64_t)a.H * TC_G, a.L, a.B)) != OK) return rc;
  ORBIT_CHECK_CUDA(cudaFuncSetAttribute(tc_chunk_out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_OUT));
  tc_chunk_out_kernel<<<dim3(a.nc, a.B), TC_THREADS, SMEM_OUT, st>>>(tmB, tmC, tmU, a);
  ORBIT_CHECK_LAUNCH("tc_chunk_out_kernel");
  return OK;
}

int tc_launch_chunk_grads(const ScanArgs&, cudaStream_t) { return fail(ERR_UNSUPPORTED, "precision 'io' backward tiles not built"); }

}  // namespace orbit

// HybridMamba clock tail: the per-token clocks and angle feature of the coordinate scan from the token slab columns.
//
//   delta[m,h] = softplus(dt_raw[m,h] + dt_bias[h])            (threshold 20, as torch.nn.functional.softplus)
//   lam[m,h]   = sigmoid(trap_raw[m,h] + trap_bias[h])         (trapezoid write only)
//   feat[m,k]  = omega[j] tanh(th_raw[m,j]) at k = rot_idx[j], 0 at the other row pairs
//
// Replaces the reference's `_fused_hm_tails` clock part (src/orbit_ssm/ssm/hybrid_mamba.py:1890-1931: `dt_softplus_cf`,
// src/orbit_ssm/layers/tails.py:1086), its angle feature (`_theta_feature`, hybrid_mamba.py:971-1000) and the exact
// sigmoid of the trapezoid weight (src/orbit_ssm/layers/layout.py:115-148).  Inputs are slab columns [M, .] in the IO
// dtype with their own row strides (read in place from the fused projection's output); outputs are fp32.  Backward
// writes the raw gradients in the IO dtype straight into their column ranges and reduces the three parameter-shaped
// gradients (dt_bias, trap_bias, omega) in two fixed-order stages: bitwise reproducible, no atomics.
// HBM-bound by construction and launch-latency sized (a few MB per call).
#include "common.cuh"
#include "../../include/orbit_b200.h"

namespace orbit {

using TailArgs = ::orbit_hm_tail_args;
constexpr int HT_THREADS = 256;          // 8 warps, one row per warp at a time
constexpr int HT_MAX_SLOTS = 148 * 4;
constexpr int HT_MAX_GROUPS = 16;        // per-lane accumulators: up to 512 parameter columns (2 H + Krot)

// full-precision forms: these clocks steer every decay of the scan, and the kernel is nowhere near an issue bound
__device__ __forceinline__ float softplus20(float v) { return v > 20.f ? v : log1pf(expf(v)); }
__device__ __forceinline__ float sigmoid_full(float v) { return 1.f / (1.f + expf(-v)); }

template <typename T>
__global__ void __launch_bounds__(HT_THREADS) hm_tail_fwd_kernel(const TailArgs a) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t nw = (int64_t)gridDim.x * (HT_THREADS / 32);
  for (int64_t m = (int64_t)blockIdx.x * (HT_THREADS / 32) + warp; m < a.M; m += nw) {
    const T* dt = (const T*)a.dt_raw + m * a.dt_rs;
    for (int h = lane; h < a.H; h += 32) a.delta[m * a.H + h] = softplus20(ldf(dt + h) + a.dt_bias[h]);
    if (a.trap_raw != nullptr) {
      const T* tr = (const T*)a.trap_raw + m * a.trap_rs;
      for (int h = lane; h < a.H; h += 32) a.lam[m * a.H + h] = sigmoid_full(ldf(tr + h) + (a.trap_bias ? a.trap_bias[h] : 0.f));
    }
    if (a.th_raw != nullptr) {
      const T* th = (const T*)a.th_raw + m * a.th_rs;
      float* f = a.feat + m * a.K;
      for (int k = lane; k < a.K; k += 32) f[k] = 0.f;
      __syncwarp();
      for (int j = lane; j < a.Krot; j += 32) f[a.rot_idx[j]] = a.omega[j] * tanhf(ldf(th + j));
    }
  }
}

// Backward.  Column c of the parameter gradients: [0, H) dt_bias, [H, 2H) trap_bias, [2H, 2H + Krot) omega.  A lane owns
// the columns congruent to it modulo 32 and sums them over the rows its warp walks; the 8 warps of a CTA are added in
// order into part[cta][2H + Krot]; hm_tail_colsum adds the CTAs in order.
template <typename T>
__global__ void __launch_bounds__(HT_THREADS) hm_tail_bwd_kernel(const TailArgs a) {
  extern __shared__ float red[];                     // [8][ncol]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int H = a.H, ncol = 2 * H + a.Krot;
  float acc[HT_MAX_GROUPS];
#pragma unroll
  for (int g = 0; g < HT_MAX_GROUPS; ++g) acc[g] = 0.f;
  const int64_t nw = (int64_t)gridDim.x * (HT_THREADS / 32);
  for (int64_t m = (int64_t)blockIdx.x * (HT_THREADS / 32) + warp; m < a.M; m += nw) {
#pragma unroll
    for (int g = 0; g < HT_MAX_GROUPS; ++g) {
      const int c = g * 32 + lane;
      if (c >= ncol) break;
      float gsum = 0.f;
      if (c < H) {
        const float v = ldf((const T*)a.dt_raw + m * a.dt_rs + c) + a.dt_bias[c];
        const float gr = (a.ddelta ? a.ddelta[m * H + c] : 0.f) * (v > 20.f ? 1.f : sigmoid_full(v));
        if (a.d_dt_raw) stf((T*)a.d_dt_raw + m * a.d_dt_rs + c, gr);
        gsum = gr;
      } else if (c < 2 * H) {
        const int h = c - H;
        if (a.trap_raw != nullptr) {
          const float l = a.lam[m * H + h];
          const float gr = (a.dlam ? a.dlam[m * H + h] : 0.f) * l * (1.f - l);
          if (a.d_trap_raw) stf((T*)a.d_trap_raw + m * a.d_trap_rs + h, gr);
          gsum = gr;
        }
      } else {
        const int j = c - 2 * H;
        if (a.th_raw != nullptr) {
          const float th = tanhf(ldf((const T*)a.th_raw + m * a.th_rs + j));
          const float gf = a.dfeat ? a.dfeat[m * a.K + a.rot_idx[j]] : 0.f;
          if (a.d_th_raw) stf((T*)a.d_th_raw + m * a.d_th_rs + j, gf * a.omega[j] * (1.f - th * th));
          gsum = gf * th;
        }
      }
      acc[g] += gsum;
    }
  }
#pragma unroll
  for (int g = 0; g < HT_MAX_GROUPS; ++g) {
    const int c = g * 32 + lane;
    if (c < ncol) red[warp * ncol + c] = acc[g];
  }
  __syncthreads();
  for (int c = threadIdx.x; c < ncol; c += HT_THREADS) {
    float v = red[c];
#pragma unroll
    for (int w = 1; w < HT_THREADS / 32; ++w) v += red[w * ncol + c];
    a.part[(int64_t)blockIdx.x * ncol + c] = v;
  }
}

__global__ void hm_tail_colsum(const float* __restrict__ part, int slots, int H, int Krot, float* __restrict__ d_dt_bias,
                               float* __restrict__ d_trap_bias, float* __restrict__ d_omega) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x, ncol = 2 * H + Krot;
  if (c >= ncol) return;
  float v = 0.f;
  for (int s = 0; s < slots; ++s) v += part[(int64_t)s * ncol + c];
  if (c < H) { if (d_dt_bias) d_dt_bias[c] = v; }
  else if (c < 2 * H) { if (d_trap_bias) d_trap_bias[c - H] = v; }
  else if (d_omega) d_omega[c - 2 * H] = v;
}

static int tail_slots(int64_t M) {
  const int64_t rows_per_cta = HT_THREADS / 32;
  const int64_t need = (M + rows_per_cta - 1) / rows_per_cta;
  return (int)(need < 1 ? 1 : (need > HT_MAX_SLOTS ? HT_MAX_SLOTS : need));
}

static int tail_check(const TailArgs* a, int dtype, const char* who, bool fwd) {
  ORBIT_REQUIRE(a != nullptr, ERR_BAD_ARG, "%s: null argument block", who);
  ORBIT_REQUIRE(dtype == F32 || dtype == BF16, ERR_BAD_ARG, "%s: unknown dtype code %d", who, dtype);
  ORBIT_REQUIRE(a->M >= 0 && a->H > 0 && a->K >= 0 && a->Krot >= 0 && a->Krot <= a->K, ERR_BAD_ARG,
                "%s: bad sizes M=%lld H=%d K=%d Krot=%d", who, (long long)a->M, a->H, a->K, a->Krot);
  ORBIT_REQUIRE(a->dt_raw && a->dt_bias, ERR_BAD_ARG, "%s: null dt_raw/dt_bias", who);
  ORBIT_REQUIRE(a->trap_raw == nullptr || a->lam != nullptr, ERR_BAD_ARG, "%s: lam is required with trap_raw", who);
  ORBIT_REQUIRE(a->th_raw == nullptr || (a->omega && a->rot_idx && a->Krot > 0), ERR_BAD_ARG,
                "%s: omega and rot_idx are required with th_raw", who);
  ORBIT_REQUIRE(!fwd || (a->delta != nullptr && (a->th_raw == nullptr || a->feat != nullptr)), ERR_BAD_ARG, "%s: null delta/feat", who);
  ORBIT_REQUIRE(2 * a->H + a->Krot <= 32 * HT_MAX_GROUPS, ERR_UNSUPPORTED,
                "%s: 2 H + Krot = %d parameter columns exceed the %d this kernel sums", who, 2 * a->H + a->Krot, 32 * HT_MAX_GROUPS);
  return OK;
}

}  // namespace orbit

using namespace orbit;

extern "C" int orbit_hm_tail_fwd(const orbit_hm_tail_args* a, int dtype, void* stream) {
  int rc = tail_check(a, dtype, "orbit_hm_tail_fwd", true);
  if (rc != OK) return rc;
  if (a->M == 0) return OK;
  const int grid = tail_slots(a->M);
  if (dtype == BF16) hm_tail_fwd_kernel<__nv_bfloat16><<<grid, HT_THREADS, 0, (cudaStream_t)stream>>>(*a);
  else hm_tail_fwd_kernel<float><<<grid, HT_THREADS, 0, (cudaStream_t)stream>>>(*a);
  ORBIT_CHECK_LAUNCH("hm_tail_fwd_kernel");
  return OK;
}

extern "C" int64_t orbit_hm_tail_bwd_workspace_bytes(int64_t M, int H, int Krot) {
  return (int64_t)tail_slots(M) * (2 * H + Krot) * (int64_t)sizeof(float);
}

extern "C" int orbit_hm_tail_bwd(const orbit_hm_tail_args* a, int dtype, void* stream) {
  int rc = tail_check(a, dtype, "orbit_hm_tail_bwd", false);
  if (rc != OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const int ncol = 2 * a->H + a->Krot;
  if (a->M == 0) {
    if (a->d_dt_bias) ORBIT_CHECK_CUDA(cudaMemsetAsync(a->d_dt_bias, 0, sizeof(float) * a->H, st));
    if (a->d_trap_bias) ORBIT_CHECK_CUDA(cudaMemsetAsync(a->d_trap_bias, 0, sizeof(float) * a->H, st));
    if (a->d_omega) ORBIT_CHECK_CUDA(cudaMemsetAsync(a->d_omega, 0, sizeof(float) * a->Krot, st));
    return OK;
  }
  ORBIT_REQUIRE(a->part != nullptr && a->part_bytes >= orbit_hm_tail_bwd_workspace_bytes(a->M, a->H, a->Krot), ERR_WORKSPACE,
                "orbit_hm_tail_bwd: workspace of %lld bytes needed", (long long)orbit_hm_tail_bwd_workspace_bytes(a->M, a->H, a->Krot));
  const int grid = tail_slots(a->M);
  const size_t smem = sizeof(float) * (HT_THREADS / 32) * ncol;
  if (dtype == BF16) hm_tail_bwd_kernel<__nv_bfloat16><<<grid, HT_THREADS, smem, st>>>(*a);
  else hm_tail_bwd_kernel<float><<<grid, HT_THREADS, smem, st>>>(*a);
  ORBIT_CHECK_LAUNCH("hm_tail_bwd_kernel");
  hm_tail_colsum<<<(ncol + 127) / 128, 128, 0, st>>>(a->part, grid, a->H, a->Krot, a->d_dt_bias, a->d_trap_bias, a->d_omega);
  ORBIT_CHECK_LAUNCH("hm_tail_colsum");
  return OK;
}

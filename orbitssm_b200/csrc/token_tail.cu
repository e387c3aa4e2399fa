// Token tails of the SSD-MIMO layer: the per-token coefficient maps between the input GEMM and the scan.
//
// Replaces the reference's `token_law` (src/orbit_ssm/ssm/ssd_mimo_torch.py:161-267; its fused CUDA form is
// `token_tails`, src/orbit_ssm/layers/tails.py:829) with two HBM-bound kernels per direction:
//   map tail    out[m, x, n] = rmsnorm_N(src[m, n*X + x]) * weight[n] + bias[n] + add        (B / C maps; gates: add = 1)
//   clock tail  dt = softplus(dt_raw), rate (static exp(A_log) | heavy-tail | softplus of a_raw), dA = -dt rate,
//               trapezoid lam = sigmoid(trap_raw): lag = dt (1 - lam), wd = lam dt, w_t = wd_t + lag_{t+1},
//               chi = r_mix + rmix_raw
// The slab columns are read in place (row strides), the gradients are written in place into the gradient of the slab.
// Parameter gradients (norm weight, shared bias, A_log, r_mix) are two-stage sums in a fixed order: no atomics.
#include "common.cuh"
#include "../../include/orbit_b200.h"

namespace orbit {

constexpr int TT_WARPS = 8;
constexpr int TT_SLOTS = 148 * 4;     // blocks of the gradient kernels (each owns one partial-sum slot)

// ------------------------------------------------------------------------------------------------------------------
// map tail
// ------------------------------------------------------------------------------------------------------------------
// One warp per (row m, sub-row x): lane handles n = lane, lane + 32, ...  (N <= 256)
template <typename T, int NV>
__global__ void __launch_bounds__(TT_WARPS * 32) map_fwd_kernel(const T* __restrict__ src, int64_t rs, const float* __restrict__ weight,
                                                                const float* __restrict__ bias, float add, float eps,
                                                                T* __restrict__ out, float* __restrict__ rstd, int64_t MX, int X, int N) {
  const int lane = threadIdx.x & 31;
  const int64_t sub = (int64_t)blockIdx.x * TT_WARPS + (threadIdx.x >> 5);
  if (sub >= MX) return;
  const int64_t m = sub / X;
  const int x = (int)(sub % X);
  float v[NV];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int n = lane + 32 * i;
    v[i] = n < N ? ldf(src + m * rs + (int64_t)n * X + x) : 0.f;
    ss = fmaf(v[i], v[i], ss);
  }
  float r = 1.f;
  if (weight != nullptr) {
    ss = warp_sum(ss);
    r = rsqrtf(ss / (float)N + eps);
    if (lane == 0) rstd[sub] = r;
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int n = lane + 32 * i;
    if (n < N) {
      float o = weight ? v[i] * r * weight[n] : v[i];
      if (bias) o += bias[n];
      stf(out + sub * N + n, o + add);
    }
  }
}

// Fixed grid; every block walks sub-rows with a grid stride and keeps its partial sums of dweight / dbias in registers.
template <typename T, int NV>
__global__ void __launch_bounds__(TT_WARPS * 32) map_bwd_kernel(const T* __restrict__ src, int64_t rs, const float* __restrict__ weight,
                                                                const float* __restrict__ rstd, const T* __restrict__ dout,
                                                                T* __restrict__ dsrc, int64_t drs, float* __restrict__ part,
                                                                int64_t MX, int X, int N, int want_dbias) {
  __shared__ float red[TT_WARPS][2][256];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float aw[NV], ab[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) { aw[i] = 0.f; ab[i] = 0.f; }
  for (int64_t sub = (int64_t)blockIdx.x * TT_WARPS + warp; sub < MX; sub += (int64_t)gridDim.x * TT_WARPS) {
    const int64_t m = sub / X;
    const int x = (int)(sub % X);
    float g[NV], xh[NV];
    float dot = 0.f;
    const float r = weight ? rstd[sub] : 1.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int n = lane + 32 * i;
      g[i] = 0.f; xh[i] = 0.f;
      if (n < N) {
        g[i] = ldf(dout + sub * N + n);
        ab[i] += g[i];
        if (weight) {
          xh[i] = ldf(src + m * rs + (int64_t)n * X + x) * r;
          aw[i] = fmaf(g[i], xh[i], aw[i]);
          g[i] *= weight[n];
          dot = fmaf(g[i], xh[i], dot);
        }
      }
    }
    if (weight) dot = warp_sum(dot) / (float)N;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int n = lane + 32 * i;
      if (n < N) stf(dsrc + m * drs + (int64_t)n * X + x, weight ? r * (g[i] - xh[i] * dot) : g[i]);
    }
  }
  if (part == nullptr) return;
#pragma unroll
  for (int i = 0; i < NV; ++i) { red[warp][0][lane + 32 * i] = aw[i]; red[warp][1][lane + 32 * i] = ab[i]; }
  __syncthreads();
  for (int idx = threadIdx.x; idx < 2 * N; idx += blockDim.x) {
    const int q = idx / N, n = idx % N;
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < TT_WARPS; ++w) s += red[w][q][n];
    part[((int64_t)blockIdx.x * 2 + q) * N + n] = s;
  }
  (void)want_dbias;
}

__global__ void slot_sum_kernel(const float* __restrict__ part, float* __restrict__ out0, float* __restrict__ out1, int nslots, int D) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= 2 * D) return;
  const int q = c / D, n = c % D;
  float* dst = q == 0 ? out0 : out1;
  if (dst == nullptr) return;
  float acc = 0.f;
  for (int s = 0; s < nslots; ++s) acc += part[((int64_t)s * 2 + q) * D + n];
  dst[n] = acc;
}

// ------------------------------------------------------------------------------------------------------------------
// clock tail
// ------------------------------------------------------------------------------------------------------------------
using ClockArgs = ::orbit_clock_args;

__device__ __forceinline__ float softplus20(float x) { return x > 20.f ? x : log1pf(__expf(x)); }
__device__ __forceinline__ float dsoftplus20(float x) { return x > 20.f ? 1.f : sigmoidf_(x); }

// rate magnitude and its derivative with respect to the raw value (boundary-passing subgradients of the clamps)
__device__ __forceinline__ void rate_act(int act, float v, float& mag, float& dmag) {
  if (act == 1) {                                   // heavy tail: 1 + v (v >= 0), 1 / (1 - v) (v <= 0), floor 1e-4
    const float inv = 1.f / (1.f - fminf(v, 0.f));
    mag = fmaxf(v, 0.f) + inv;
    dmag = (v >= 0.f ? 1.f : 0.f) + (v <= 0.f ? inv * inv : 0.f);
  } else {                                          // softplus, floor 1e-4
    mag = softplus20(v);
    dmag = dsoftplus20(v);
  }
  if (mag < 1e-4f) { mag = 1e-4f; dmag = 0.f; }
}

template <typename T>
__global__ void __launch_bounds__(256) clock_fwd_kernel(const ClockArgs a) {
  const int HR = a.H * a.R;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= a.M * HR) return;
  int64_t m;
  int hr, t;
  if (a.M * HR < (int64_t)1 << 31) {          // the usual case: 32-bit index splits (a 64-bit division costs ~5 x as much)
    const uint32_t i32 = (uint32_t)idx, m32 = i32 / (uint32_t)HR;
    m = m32;
    hr = (int)(i32 - m32 * (uint32_t)HR);
    t = (int)(m32 % (uint32_t)a.L);
  } else {
    m = idx / HR;
    hr = (int)(idx % HR);
    t = (int)(m % a.L);
  }
  const int h = hr / a.R;
  const T* dtp = (const T*)a.dt_raw;
  const float dt = softplus20(ldf(dtp + m * a.dt_rs + hr));
  float rate;
  if (a.a_act == 0) rate = __expf(a.A_log[hr]);
  else {
    float dm;
    rate_act(a.a_act, ldf((const T*)a.a_raw + m * a.a_rs + (a.a_per_sibling ? hr : h)), rate, dm);
  }
  a.dA[idx] = -dt * rate;
  if (a.trap_raw != nullptr) {
    const T* tp = (const T*)a.trap_raw;
    const float lam = sigmoidf_(ldf(tp + m * a.trap_rs + h));
    float lag_next = 0.f;
    if (t + 1 < a.L) {
      const float dtn = softplus20(ldf(dtp + (m + 1) * a.dt_rs + hr));
      lag_next = dtn * (1.f - sigmoidf_(ldf(tp + (m + 1) * a.trap_rs + h)));
    }
    const float wd = lam * dt;
    a.wd[idx] = wd;
    a.w[idx] = wd + lag_next;
    if (t == 0 && a.lag0 != nullptr) a.lag0[(m / a.L) * HR + hr] = dt * (1.f - lam);
  } else {
    a.w[idx] = dt;
  }
  if (a.chi != nullptr) a.chi[idx] = a.r_mix[hr] + (a.rmix_raw ? ldf((const T*)a.rmix_raw + m * a.rmix_rs + hr) : 0.f);
}

// One thread per (row m, head h): loops the R siblings so that the per-head raw gradients (trap, shared a) are summed in
// a fixed order by their single owner.  With a static rate the per-element term of dA_log goes to g_alog [M, H*R]
// (the caller sums it over rows); d r_mix is the row sum of dchi and needs no kernel.
// The grid strides over the rows by a multiple of H, so a thread keeps its head and can sum the UNROUNDED raw gradients
// of its rows in registers: these column sums are the gradients of the slab biases (dt, a, trap), exact in fp32 where a
// sum over the bf16-rounded slab gradient would carry the rounding of every row.  Per-CTA sums (threads of a head added
// in thread order) go to sum_part [gridDim.x][ncol]; clock_colsum_kernel adds the CTAs in order.
constexpr int CLK_MAXR = 4;      // = the rank limit of the scan argument block

__host__ __device__ inline int clock_sum_cols(int H, int R, int a_act, int a_per_sibling, bool trap) {
  return H * R + (a_act != 0 ? (a_per_sibling ? H * R : H) : 0) + (trap ? H : 0);
}

template <typename T>
__global__ void __launch_bounds__(256, 3) clock_bwd_kernel(const ClockArgs a) {
  __shared__ float sacc[2 * CLK_MAXR + 1][256];
  const int HR = a.H * a.R;
  const T* dtp = (const T*)a.dt_raw;
  const T* tp = (const T*)a.trap_raw;
  const int64_t total = a.M * a.H, stride = (int64_t)gridDim.x * blockDim.x;
  float acc_dt[CLK_MAXR], acc_a[CLK_MAXR], acc_trap = 0.f;
#pragma unroll
  for (int r = 0; r < CLK_MAXR; ++r) { acc_dt[r] = 0.f; acc_a[r] = 0.f; }
  // The stride is a multiple of H (the launch sees to it), so the thread keeps its head: row and token advance by fixed
  // steps, and the divisions of the flat index are paid once, not per element.
  const int64_t e0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool keeps_head = stride % a.H == 0;
  int64_t m = e0 / a.H;
  int h = (int)(e0 % a.H);
  int t = (int)(m % a.L);
  const int64_t dm = stride / a.H;
  const int dtl = (int)(dm % a.L);
  float rate_c[CLK_MAXR];
#pragma unroll
  for (int r = 0; r < CLK_MAXR; ++r) rate_c[r] = (a.a_act == 0 && r < a.R) ? __expf(a.A_log[h * a.R + r]) : 0.f;
  for (int64_t e = e0; e < total; e += stride, m += dm, t = t + dtl >= a.L ? t + dtl - a.L : t + dtl) {
    if (!keeps_head) {
      m = e / a.H;
      h = (int)(e % a.H);
      t = (int)(m % a.L);
    }
    float lam = 1.f;
    if (tp != nullptr) lam = sigmoidf_(ldf(tp + m * a.trap_rs + h));
    float g_trap = 0.f, g_ah = 0.f;
#pragma unroll
    for (int r = 0; r < CLK_MAXR; ++r) {
      if (r >= a.R) break;
      const int hr = h * a.R + r;
      const int64_t idx = m * HR + hr;
      const float raw = ldf(dtp + m * a.dt_rs + hr);
      const float dt = softplus20(raw);
      float rate, dmag = 0.f;
      if (a.a_act == 0) rate = keeps_head ? rate_c[r] : __expf(a.A_log[hr]);
      else rate_act(a.a_act, ldf((const T*)a.a_raw + m * a.a_rs + (a.a_per_sibling ? hr : h)), rate, dmag);
      const float gdA = a.ddA[idx];
      float g_dt = -gdA * rate;
      const float g_rate = -gdA * dt;
      if (a.a_act == 0) a.g_alog[idx] = g_rate * rate;
      else if (a.a_per_sibling) {
        stf((T*)a.d_a_raw + m * a.da_rs + hr, g_rate * dmag);
        acc_a[r] += g_rate * dmag;
      } else g_ah = fmaf(g_rate, dmag, g_ah);
      if (tp != nullptr) {
        // w_t = lam_t dt_t + lag_{t+1};  lag_t = dt_t (1 - lam_t) enters w_{t-1} (and lag0 at t = 0)
        const float gsum = a.dw[idx] + (a.dwd ? a.dwd[idx] : 0.f);
        float glag = 0.f;
        if (t > 0) glag = a.dw[idx - HR];
        else if (a.dlag0 != nullptr) glag = a.dlag0[(m / a.L) * HR + hr];
        g_dt += gsum * lam + glag * (1.f - lam);
        g_trap = fmaf((gsum - glag) * dt, lam * (1.f - lam), g_trap);
      } else {
        g_dt += a.dw[idx];
      }
      const float g_raw = g_dt * dsoftplus20(raw);
      stf((T*)a.d_dt_raw + m * a.ddt_rs + hr, g_raw);
      acc_dt[r] += g_raw;
      if (a.d_rmix_raw != nullptr) stf((T*)a.d_rmix_raw + m * a.drmix_rs + hr, a.dchi ? a.dchi[idx] : 0.f);
    }
    if (tp != nullptr) {
      stf((T*)a.d_trap_raw + m * a.dtrap_rs + h, g_trap);
      acc_trap += g_trap;
    }
    if (a.a_act != 0 && !a.a_per_sibling) {
      stf((T*)a.d_a_raw + m * a.da_rs + h, g_ah);
      acc_a[0] += g_ah;
    }
  }
  if (a.sum_part == nullptr) return;
  // ---- per-CTA column sums: thread i holds head (blockIdx.x * 256 + i) mod H
#pragma unroll
  for (int r = 0; r < CLK_MAXR; ++r) {
    sacc[r][threadIdx.x] = acc_dt[r];
    sacc[CLK_MAXR + r][threadIdx.x] = acc_a[r];
  }
  sacc[2 * CLK_MAXR][threadIdx.x] = acc_trap;
  __syncthreads();
  const int ncol = clock_sum_cols(a.H, a.R, a.a_act, a.a_per_sibling, tp != nullptr);
  const int off_a = HR, off_t = HR + (a.a_act != 0 ? (a.a_per_sibling ? HR : a.H) : 0);
  float* part = a.sum_part + (int64_t)blockIdx.x * ncol;
  const int phase = (int)(((int64_t)blockIdx.x * blockDim.x) % a.H);
  for (int h = threadIdx.x; h < a.H; h += blockDim.x) {
    const int i0 = ((h - phase) % a.H + a.H) % a.H;      // first thread of this CTA that holds head h
    float sdt[CLK_MAXR], sa[CLK_MAXR], st = 0.f;
#pragma unroll
    for (int r = 0; r < CLK_MAXR; ++r) { sdt[r] = 0.f; sa[r] = 0.f; }
    for (int i = i0; i < (int)blockDim.x; i += a.H) {
#pragma unroll
      for (int r = 0; r < CLK_MAXR; ++r) { sdt[r] += sacc[r][i]; sa[r] += sacc[CLK_MAXR + r][i]; }
      st += sacc[2 * CLK_MAXR][i];
    }
    for (int r = 0; r < a.R; ++r) {
      part[h * a.R + r] = sdt[r];
      if (a.a_act != 0 && a.a_per_sibling) part[off_a + h * a.R + r] = sa[r];
    }
    if (a.a_act != 0 && !a.a_per_sibling) part[off_a + h] = sa[0];
    if (tp != nullptr) part[off_t + h] = st;
  }
}

// out[c] = sum over the CTAs' partial sums in a fixed order: a CTA owns 32 columns, warp g adds the slots congruent to g
// modulo 8, then the 8 sums are added in order.
__global__ void __launch_bounds__(256) clock_colsum_kernel(const float* __restrict__ part, int slots, int ncol, float* __restrict__ out) {
  __shared__ float red[8][33];
  const int lane = threadIdx.x & 31, grp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float acc = 0.f;
  if (c < ncol) {
#pragma unroll 4
    for (int s = grp; s < slots; s += 8) acc += part[(int64_t)s * ncol + c];
  }
  red[grp][lane] = acc;
  __syncthreads();
  if (grp == 0 && c < ncol) {
    float v = red[0][lane];
#pragma unroll
    for (int g = 1; g < 8; ++g) v += red[g][lane];
    out[c] = v;
  }
}

// CTAs of the backward: a multiple of H / gcd(256, H), so that the grid stride is a multiple of H
static int clock_bwd_grid(int64_t M, int H) {
  int g = 256, hh = H;
  while (hh) { const int tmp = g % hh; g = hh; hh = tmp; }       // g = gcd(256, H)
  const int unit = H / g;
  const int64_t need = (M * H + 255) / 256;
  int64_t cap = 148 * 3;            // what is resident at once (three CTAs per SM by the launch bounds): one even wave
  if (need < cap) cap = need;
  int64_t grid = (cap / unit) * unit;
  if (grid < unit) grid = unit;
  return (int)grid;
}

static int map_nv(int N) { return (N + 31) / 32; }

}  // namespace orbit

using namespace orbit;

extern "C" int64_t orbit_token_map_bwd_workspace_bytes(int N) { return (int64_t)TT_SLOTS * 2 * N * (int64_t)sizeof(float); }

extern "C" int orbit_token_map_fwd(const void* src, int64_t src_row_stride, const float* weight, const float* bias, float add,
                                   float eps, void* out, float* rstd, int64_t M, int X, int N, int dtype, void* stream) {
  ORBIT_REQUIRE(src && out, ERR_BAD_ARG, "orbit_token_map_fwd: null src/out");
  ORBIT_REQUIRE(dtype == F32 || dtype == BF16, ERR_BAD_ARG, "orbit_token_map_fwd: unknown dtype code %d", dtype);
  ORBIT_REQUIRE(M >= 0 && X >= 1 && N >= 1 && N <= 256, ERR_UNSUPPORTED, "orbit_token_map_fwd: serves 1 <= N <= 256, X >= 1 (M=%lld X=%d N=%d)",
                (long long)M, X, N);
  ORBIT_REQUIRE(weight == nullptr || rstd != nullptr, ERR_BAD_ARG, "orbit_token_map_fwd: rstd is required with a norm weight");
  if (M == 0) return OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t MX = M * X;
  const int grid = (int)((MX + TT_WARPS - 1) / TT_WARPS);
#define L_(TY, NV) map_fwd_kernel<TY, NV><<<grid, TT_WARPS * 32, 0, st>>>((const TY*)src, src_row_stride, weight, bias, add, eps, (TY*)out, rstd, MX, X, N)
  const int nv = map_nv(N);
  if (dtype == BF16) { if (nv <= 1) L_(__nv_bfloat16, 1); else if (nv <= 2) L_(__nv_bfloat16, 2); else if (nv <= 4) L_(__nv_bfloat16, 4); else L_(__nv_bfloat16, 8); }
  else { if (nv <= 1) L_(float, 1); else if (nv <= 2) L_(float, 2); else if (nv <= 4) L_(float, 4); else L_(float, 8); }
#undef L_
  ORBIT_CHECK_LAUNCH("map_fwd_kernel");
  return OK;
}

extern "C" int orbit_token_map_bwd(const void* src, int64_t src_row_stride, const float* weight, const float* rstd, const void* dout,
                                   void* dsrc, int64_t dsrc_row_stride, float* dweight, float* dbias, void* workspace,
                                   int64_t workspace_bytes, int64_t M, int X, int N, int dtype, void* stream) {
  ORBIT_REQUIRE(dout && dsrc, ERR_BAD_ARG, "orbit_token_map_bwd: null dout/dsrc");
  ORBIT_REQUIRE(dtype == F32 || dtype == BF16, ERR_BAD_ARG, "orbit_token_map_bwd: unknown dtype code %d", dtype);
  ORBIT_REQUIRE(M >= 0 && X >= 1 && N >= 1 && N <= 256, ERR_UNSUPPORTED, "orbit_token_map_bwd: serves 1 <= N <= 256, X >= 1");
  ORBIT_REQUIRE(weight == nullptr || (src && rstd && dweight), ERR_BAD_ARG, "orbit_token_map_bwd: src, rstd, dweight are required with a norm weight");
  const bool sums = dweight != nullptr || dbias != nullptr;
  ORBIT_REQUIRE(!sums || (workspace && workspace_bytes >= orbit_token_map_bwd_workspace_bytes(N)), ERR_WORKSPACE,
                "orbit_token_map_bwd: workspace of %lld bytes needed", (long long)orbit_token_map_bwd_workspace_bytes(N));
  cudaStream_t st = (cudaStream_t)stream;
  if (M == 0) {
    if (dweight) ORBIT_CHECK_CUDA(cudaMemsetAsync(dweight, 0, N * sizeof(float), st));
    if (dbias) ORBIT_CHECK_CUDA(cudaMemsetAsync(dbias, 0, N * sizeof(float), st));
    return OK;
  }
  const int64_t MX = M * X;
  int grid = (int)((MX + TT_WARPS - 1) / TT_WARPS);
  if (grid > TT_SLOTS) grid = TT_SLOTS;
  float* part = sums ? (float*)workspace : nullptr;
#define L_(TY, NV) map_bwd_kernel<TY, NV><<<grid, TT_WARPS * 32, 0, st>>>((const TY*)src, src_row_stride, weight, rstd, (const TY*)dout, (TY*)dsrc, dsrc_row_stride, part, MX, X, N, dbias != nullptr)
  const int nv = map_nv(N);
  if (dtype == BF16) { if (nv <= 1) L_(__nv_bfloat16, 1); else if (nv <= 2) L_(__nv_bfloat16, 2); else if (nv <= 4) L_(__nv_bfloat16, 4); else L_(__nv_bfloat16, 8); }
  else { if (nv <= 1) L_(float, 1); else if (nv <= 2) L_(float, 2); else if (nv <= 4) L_(float, 4); else L_(float, 8); }
#undef L_
  ORBIT_CHECK_LAUNCH("map_bwd_kernel");
  if (sums) {
    slot_sum_kernel<<<(2 * N + 255) / 256, 256, 0, st>>>(part, dweight, dbias, grid, N);
    ORBIT_CHECK_LAUNCH("slot_sum_kernel");
  }
  return OK;
}

static int clock_check(const orbit_clock_args* a, int dtype, const char* who, bool bwd) {
  ORBIT_REQUIRE(a != nullptr, ERR_BAD_ARG, "%s: null argument block", who);
  ORBIT_REQUIRE(dtype == F32 || dtype == BF16, ERR_BAD_ARG, "%s: unknown dtype code %d", who, dtype);
  ORBIT_REQUIRE(a->M >= 0 && a->L > 0 && a->H > 0 && a->R > 0 && a->M % a->L == 0, ERR_BAD_ARG, "%s: bad sizes M=%lld L=%d H=%d R=%d", who,
                (long long)a->M, a->L, a->H, a->R);
  ORBIT_REQUIRE(a->dt_raw != nullptr, ERR_BAD_ARG, "%s: null dt_raw", who);
  ORBIT_REQUIRE(a->a_act >= 0 && a->a_act <= 2 && (a->a_act == 0 ? a->A_log != nullptr : a->a_raw != nullptr), ERR_BAD_ARG,
                "%s: a_act 0 needs A_log, a_act 1 / 2 need a_raw", who);
  if (!bwd) {
    ORBIT_REQUIRE(a->dA && a->w && (a->trap_raw == nullptr || a->wd != nullptr) && (a->chi == nullptr || a->r_mix != nullptr), ERR_BAD_ARG,
                  "%s: null dA/w (or wd with a trapezoid, r_mix with chi)", who);
  } else {
    ORBIT_REQUIRE(a->ddA && a->dw && a->d_dt_raw && (a->a_act != 0 || a->g_alog) && (a->a_act == 0 || a->d_a_raw) &&
                      (a->trap_raw == nullptr || a->d_trap_raw),
                  ERR_BAD_ARG, "%s: null ddA/dw/d_dt_raw (or g_alog / d_a_raw / d_trap_raw for the options in use)", who);
  }
  return OK;
}

extern "C" int orbit_token_clock_fwd(const orbit_clock_args* a, int dtype, void* stream) {
  int rc = clock_check(a, dtype, "orbit_token_clock_fwd", false);
  if (rc != OK) return rc;
  if (a->M == 0) return OK;
  const int64_t n = a->M * a->H * a->R;
  const int grid = (int)((n + 255) / 256);
  if (dtype == BF16) clock_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>(*a);
  else clock_fwd_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>(*a);
  ORBIT_CHECK_LAUNCH("clock_fwd_kernel");
  return OK;
}

extern "C" int64_t orbit_token_clock_bwd_workspace_bytes(int64_t M, int H, int R, int a_act, int a_per_sibling, int trap) {
  if (M <= 0 || H <= 0 || R <= 0) return 0;
  return (int64_t)clock_bwd_grid(M, H) * clock_sum_cols(H, R, a_act, a_per_sibling, trap != 0) * (int64_t)sizeof(float);
}

extern "C" int orbit_token_clock_bwd(const orbit_clock_args* a, int dtype, void* stream) {
  int rc = clock_check(a, dtype, "orbit_token_clock_bwd", true);
  if (rc != OK) return rc;
  if (a->M == 0) return OK;
  ORBIT_REQUIRE(a->R <= CLK_MAXR, ERR_UNSUPPORTED, "orbit_token_clock_bwd: ranks up to %d are served, got R=%d", CLK_MAXR, a->R);
  const int grid = clock_bwd_grid(a->M, a->H);
  const int ncol = clock_sum_cols(a->H, a->R, a->a_act, a->a_per_sibling, a->trap_raw != nullptr);
  if (a->sum_part != nullptr) {
    ORBIT_REQUIRE(a->bias_sums != nullptr && a->sum_part_bytes >= orbit_token_clock_bwd_workspace_bytes(a->M, a->H, a->R, a->a_act,
                                                                                                   a->a_per_sibling, a->trap_raw != nullptr),
                  ERR_WORKSPACE, "orbit_token_clock_bwd: bias_sums and a workspace of %lld bytes are needed for the column sums",
                  (long long)orbit_token_clock_bwd_workspace_bytes(a->M, a->H, a->R, a->a_act, a->a_per_sibling, a->trap_raw != nullptr));
  }
  if (dtype == BF16) clock_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>(*a);
  else clock_bwd_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>(*a);
  ORBIT_CHECK_LAUNCH("clock_bwd_kernel");
  if (a->sum_part != nullptr) {
    clock_colsum_kernel<<<(ncol + 31) / 32, 256, 0, (cudaStream_t)stream>>>(a->sum_part, grid, ncol, a->bias_sums);
    ORBIT_CHECK_LAUNCH("clock_colsum_kernel");
  }
  return OK;
}

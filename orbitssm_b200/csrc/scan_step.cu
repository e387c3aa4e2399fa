// SSD-MIMO scan, one token (decode): the law of the chunked scan at L = 1 in ONE launch, any (R, O, G, N).
//
//   v[g,r,n]   = sum_q u[g,q] Bbar_r[q,n]                          the folded write of the token
//   S'[r,n,g]  = exp(dA_r) S[r,n,g] + w_r v[g,r,n]                 state after the token (fp32, kernel layout [B,H,R,N,G])
//   y[g,o]     = sum_r chi_r ( sum_n Cbar_r[o,n] (exp(dA_r) S[r,n,g] + wd_r v[g,r,n]) + D[h,g,r,o] u[g,r] )
//
// with Bbar_r[q,n] = gBp[r,n] Bhat[q,n] + beta[h,r,q,n], Cbar_r[o,n] = gCp[o,n] Chat[o,n] + gamma[h,r,o,n]: exactly what
// chunk_state -> state_pass -> chunk_out compute for a one-token sequence (three launches, the tensor-core ones on a
// 128-token tile), so a sequence stepped token by token equals the sequence run at once.  Replaces the reference's
// `_step_core` inside `ssd_step` / `mixer_step_fast` (src/orbit_ssm/ssm/ssd_mimo_torch.py:388-490).  Inference only (no
// gradient).  One CTA per (batch, head); the state tile is read and written once, coalesced over the channel axis:
// HBM-bound at 8 bytes per state element per token.
#include "common.cuh"
#include "../../include/orbit_b200.h"
#include "scan_args.h"

namespace orbit {

constexpr int STEP_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(STEP_THREADS) ssd_step_kernel(const ScanArgs a, const float* __restrict__ S0, float* __restrict__ S1) {
  extern __shared__ float sm[];
  const int R = a.R, O = a.O, G = a.G, N = a.N;
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
  float* Bbar = sm;                       // [R][R q][N]
  float* Cbar = Bbar + R * R * N;         // [R][O][N]
  float* us = Cbar + R * O * N;           // [G][R]
  float* ck = us + G * R;                 // [4][R]: exp(dA), w, wd, chi
  float* rd = ck + 4 * R;                 // [R][N][G]: what the read map sees, chi folded in
  float* yp = rd + R * N * G;             // [parts][G*O]
  const T* Bh = (const T*)a.Bhat + (int64_t)b * a.b_ts;
  const T* Chh = (const T*)a.Chat + (int64_t)b * a.c_ts;
  const T* gB = a.gBp ? (const T*)a.gBp + (int64_t)b * a.gb_ts : nullptr;
  const T* gC = a.gCp ? (const T*)a.gCp + (int64_t)b * a.gc_ts : nullptr;
  for (int idx = tid; idx < R * R * N; idx += STEP_THREADS) {
    const int n = idx % N, q = (idx / N) % R, r = idx / (N * R);
    float v = ldf(Bh + q * N + n);
    if (gB) v *= ldf(gB + r * N + n);
    if (a.beta) v += a.beta[(((int64_t)h * R + r) * R + q) * N + n];
    Bbar[idx] = v;
  }
  for (int idx = tid; idx < R * O * N; idx += STEP_THREADS) {
    const int n = idx % N, o = (idx / N) % O, r = idx / (N * O);
    float v = ldf(Chh + o * N + n);
    if (gC) v *= ldf(gC + o * N + n);
    if (a.gamma) v += a.gamma[(((int64_t)h * R + r) * O + o) * N + n];
    Cbar[idx] = v;
  }
  const T* up = (const T*)a.u + ((int64_t)b * a.H + h) * G * R;
  for (int idx = tid; idx < G * R; idx += STEP_THREADS) us[idx] = ldf(up + idx);
  if (tid < R) {
    const int64_t i = ((int64_t)b * a.H + h) * R + tid;
    ck[tid] = __expf(a.dA[i]);
    ck[R + tid] = a.w[i];
    ck[2 * R + tid] = a.wd[i];
    ck[3 * R + tid] = a.chi ? a.chi[i] : 1.f;
  }
  __syncthreads();
  const int64_t sbase = ((int64_t)b * a.H + h) * R * (int64_t)N * G;
  for (int idx = tid; idx < R * N * G; idx += STEP_THREADS) {
    const int g = idx % G, n = (idx / G) % N, r = idx / (G * N);
    float v = 0.f;
    for (int q = 0; q < R; ++q) v = fmaf(us[g * R + q], Bbar[(r * R + q) * N + n], v);
    const float carried = ck[r] * (S0 ? S0[sbase + idx] : 0.f);
    S1[sbase + idx] = fmaf(ck[R + r], v, carried);
    rd[idx] = ck[3 * R + r] * fmaf(ck[2 * R + r], v, carried);
  }
  __syncthreads();
  // y[g,o]: the (r, n) sum split over `parts` thread groups, partial sums added in order
  const int GO = G * O;
  const int parts = GO >= STEP_THREADS ? 1 : STEP_THREADS / GO;
  const int RN = R * N;
  for (int base = 0; base < GO; base += STEP_THREADS) {
    const int part = (GO >= STEP_THREADS) ? 0 : tid / GO;
    const int go = (GO >= STEP_THREADS) ? base + tid : tid % GO;
    if (go < GO && part < parts) {
      const int o = go % O, g = go / O;
      float acc = 0.f;
      for (int rn = part; rn < RN; rn += parts) {
        const int n = rn % N, r = rn / N;
        acc = fmaf(Cbar[(r * O + o) * N + n], rd[(r * N + n) * G + g], acc);
      }
      yp[part * GO + go] = acc;
    }
    __syncthreads();
    if (go < GO && part == 0) {
      const int o = go % O, g = go / O;
      float acc = yp[go];
      for (int p = 1; p < parts; ++p) acc += yp[p * GO + go];
      if (a.Dg)
        for (int r = 0; r < R; ++r) acc = fmaf(ck[3 * R + r] * a.Dg[(((int64_t)h * G + g) * R + r) * O + o], us[g * R + r], acc);
      stf((T*)a.y + ((int64_t)b * a.H + h) * GO + go, acc);
    }
    __syncthreads();
    if (GO < STEP_THREADS) break;
  }
}

static size_t step_smem(const ScanArgs& a) {
  const size_t GO = (size_t)a.G * a.O;
  const size_t parts = GO >= STEP_THREADS ? 1 : STEP_THREADS / GO;
  return sizeof(float) * ((size_t)a.R * a.R * a.N + (size_t)a.R * a.O * a.N + (size_t)a.G * a.R + 4 * a.R +
                          (size_t)a.R * a.N * a.G + parts * GO);
}

}  // namespace orbit

using namespace orbit;

extern "C" int orbit_ssd_scan_step(const orbit_scan_args* a, const float* S0, float* S1, int dtype, void* stream) {
  ORBIT_REQUIRE(a != nullptr, ERR_BAD_ARG, "orbit_ssd_scan_step: null argument block");
  ORBIT_REQUIRE(dtype == F32 || dtype == BF16, ERR_BAD_ARG, "orbit_ssd_scan_step: unknown dtype code %d", dtype);
  ORBIT_REQUIRE(a->B >= 0 && a->H > 0 && a->R > 0 && a->O > 0 && a->G > 0 && a->N > 0, ERR_BAD_ARG,
                "orbit_ssd_scan_step: bad geometry B=%d H=%d R=%d O=%d G=%d N=%d", a->B, a->H, a->R, a->O, a->G, a->N);
  ORBIT_REQUIRE(a->L == 1, ERR_BAD_ARG, "orbit_ssd_scan_step: one token per call (L = %d)", a->L);
  ORBIT_REQUIRE(a->u && a->Bhat && a->Chat && a->dA && a->w && a->wd && a->y && S1, ERR_BAD_ARG,
                "orbit_ssd_scan_step: null u/Bhat/Chat/dA/w/wd/y/S1");
  if (a->B == 0) return OK;
  const size_t smem = step_smem(*a);
  ORBIT_REQUIRE(smem <= 200 * 1024, ERR_UNSUPPORTED,
                "orbit_ssd_scan_step: one head's state tile and maps need %zu bytes of shared memory (limit 204800): R=%d O=%d G=%d N=%d",
                smem, a->R, a->O, a->G, a->N);
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid(a->H, a->B);
  if (dtype == BF16) {
    ORBIT_CHECK_CUDA(cudaFuncSetAttribute(ssd_step_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    ssd_step_kernel<__nv_bfloat16><<<grid, STEP_THREADS, smem, st>>>(*a, S0, S1);
  } else {
    ORBIT_CHECK_CUDA(cudaFuncSetAttribute(ssd_step_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    ssd_step_kernel<float><<<grid, STEP_THREADS, smem, st>>>(*a, S0, S1);
  }
  ORBIT_CHECK_LAUNCH("ssd_step_kernel");
  return OK;
}

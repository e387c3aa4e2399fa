// Entry points of the SSD-MIMO scan: state pass kernels (shared by both precisions) and the phase drivers.
#include "common.cuh"
#include "scan_args.h"
#include <stdarg.h>

namespace orbit {

// ---- error text (thread-local) -------------------------------------------------------------------
static thread_local char g_err[512] = {0};
void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

// ---- state pass ------------------------------------------------------------------------------------
// Forward: buf[c] holds the chunk-local state Z[c] on entry and the state ENTERING chunk c on exit;
//   S <- S0;  for c: z = buf[c]; buf[c] = S; S = atot[c] * S + z;   S_fin <- S
// One thread per VEC state elements of one (batch, head, sibling); the walk over chunks is the only serial part of
// the scan (the reference's `_cp_pass`, src/orbit_ssm/kernels/ssd_mimo/chunkpar.py:19-25).  Loads are issued PASS_NB
// chunks ahead of the dependent multiply-add chain, so the kernel runs at memory speed, not at load latency.
// With REVERSE the walk runs from the last chunk down (the adjoint pass):
//   D <- dS_fin;  for c = nc-1..0: g = buf[c]; buf[c] = D; D = atot[c] * D + g;   dS0 <- D
// `copy16` (optional) receives a bfloat16 copy of what is written to buf (operand tiles of the tensor-core kernels).
// With WRITE32 false only that copy is written: the rank-1 tensor-core kernels read nothing but the bfloat16 tiles, so
// the fp32 write-back (40 % of this kernel's traffic) is left out and buf keeps the chunk-local values.
constexpr int PASS_NB = 8;

template <int VEC, bool REVERSE, bool WRITE, bool WRITE32>
__global__ void __launch_bounds__(256, 3) state_pass_kernel(float* __restrict__ buf, const float* __restrict__ atot,
                                                         const float* __restrict__ s_in, float* __restrict__ s_out,
                                                         __nv_bfloat16* __restrict__ copy16, int nc, int HR, int NG) {
  const int e = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  const int hr = blockIdx.y, b = blockIdx.z;
  if (e >= NG) return;
  float S[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) S[i] = s_in ? s_in[((int64_t)b * HR + hr) * NG + e + i] : 0.f;
  const int64_t base = ((int64_t)b * nc * HR + hr) * NG + e;
  const float* ap = atot + (int64_t)b * nc * HR + hr;
  const int64_t cstride = (int64_t)HR * NG;
  for (int c0 = 0; c0 < nc; c0 += PASS_NB) {
    float z[PASS_NB][VEC], av[PASS_NB];
#pragma unroll
    for (int kk = 0; kk < PASS_NB; ++kk) {
      // The loads of a batch are issued from the highest address down in both directions: measured, the forward walk ran
      // 1.45 x longer than the reverse one for the same traffic when its eight loads (2 MiB apart at the config-5 size)
      // went out lowest address first.
      const int k = REVERSE ? kk : PASS_NB - 1 - kk;
      const int cc = REVERSE ? nc - 1 - (c0 + k) : c0 + k;
      if (c0 + k < nc) {
        av[k] = ap[(int64_t)cc * HR];
        if constexpr (VEC == 4) {
          float4 v = *reinterpret_cast<const float4*>(buf + base + cc * cstride);
          z[k][0] = v.x; z[k][1] = v.y; z[k][2] = v.z; z[k][3] = v.w;
        } else {
          z[k][0] = buf[base + cc * cstride];
        }
      }
    }
#pragma unroll
    for (int k = 0; k < PASS_NB; ++k) {
      const int cc = REVERSE ? nc - 1 - (c0 + k) : c0 + k;
      if (c0 + k < nc) {
        if constexpr (!WRITE) {
          // dry walk: only the carried value is wanted (context-parallel exchange), the buffer keeps its content
        } else if constexpr (VEC == 4) {
          if constexpr (WRITE32) *reinterpret_cast<float4*>(buf + base + cc * cstride) = make_float4(S[0], S[1], S[2], S[3]);
          if (copy16) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(S[0], S[1]), hi = __floats2bfloat162_rn(S[2], S[3]);
            *reinterpret_cast<uint2*>(copy16 + base + cc * cstride) =
                make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
          }
        } else {
          if constexpr (WRITE32) buf[base + cc * cstride] = S[0];
          if (copy16) copy16[base + cc * cstride] = __float2bfloat16_rn(S[0]);
        }
#pragma unroll
        for (int i = 0; i < VEC; ++i) S[i] = fmaf(av[k], S[i], z[k][i]);
      }
    }
  }
  if (s_out) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) s_out[((int64_t)b * HR + hr) * NG + e + i] = S[i];
  }
}

template <bool REVERSE, bool WRITE, bool WRITE32>
static int launch_state_pass(float* buf, const float* atot, const float* s_in, float* s_out, void* copy16,
                             const ScanArgs& a, cudaStream_t st) {
  const int NG = a.N * a.G, HR = a.H * a.R;
  const bool vec = NG % 4 == 0 && aligned16(buf) && (copy16 == nullptr || (reinterpret_cast<uintptr_t>(copy16) & 7u) == 0);
  if (vec) {
    dim3 grid((NG / 4 + 255) / 256, HR, a.B);
    state_pass_kernel<4, REVERSE, WRITE, WRITE32><<<grid, 256, 0, st>>>(buf, atot, s_in, s_out, (__nv_bfloat16*)copy16, a.nc, HR, NG);
  } else {
    dim3 grid((NG + 255) / 256, HR, a.B);
    state_pass_kernel<1, REVERSE, WRITE, WRITE32><<<grid, 256, 0, st>>>(buf, atot, s_in, s_out, (__nv_bfloat16*)copy16, a.nc, HR, NG);
  }
  ORBIT_CHECK_LAUNCH("state_pass_kernel");
  return OK;
}

// The rank-1 tensor-core kernels (R = O = 1 with bfloat16 state tiles supplied) read the bfloat16 tiles only.
static bool tiles_only(const ScanArgs& a, const void* copy16) { return copy16 != nullptr && a.R == 1 && a.O == 1; }

int launch_state_pass_fwd(const ScanArgs& a, const float* S0, float* S_fin, cudaStream_t st, bool dry = false) {
  if (dry) return launch_state_pass<false, false, false>(a.Sin, a.atot, S0, S_fin, nullptr, a, st);
  if (tiles_only(a, a.Sin16)) return launch_state_pass<false, true, false>(a.Sin, a.atot, S0, S_fin, a.Sin16, a, st);
  return launch_state_pass<false, true, true>(a.Sin, a.atot, S0, S_fin, a.Sin16, a, st);
}

int launch_state_pass_bwd(const ScanArgs& a, const float* dS_fin, float* dS0, cudaStream_t st, bool dry = false) {
  if (dry) return launch_state_pass<true, false, false>(a.dS, a.atot, dS_fin, dS0, nullptr, a, st);
  if (tiles_only(a, a.dS16)) return launch_state_pass<true, true, false>(a.dS, a.atot, dS_fin, dS0, a.dS16, a, st);
  return launch_state_pass<true, true, true>(a.dS, a.atot, dS_fin, dS0, a.dS16, a, st);
}

// precision "ieee" phase launchers (scan_generic.cu)
int gen_pick_chunk(int R, int O, int G, int N, int backward, int limit);
int gen_launch_chunk_state(const ScanArgs& a, int dtype, cudaStream_t st);
int gen_launch_chunk_out(const ScanArgs& a, int dtype, cudaStream_t st);
int gen_launch_chunk_dstate(const ScanArgs& a, int dtype, cudaStream_t st);
int gen_launch_chunk_grads(const ScanArgs& a, int dtype, cudaStream_t st);
// precision "io" phase launchers (scan_tc.cu)
int tc_supported(const ScanArgs& a, int dtype, const char** why);
int tc_pick_chunk(int R, int O, int G, int N, int backward, int limit);
int tc_launch_chunk_state(const ScanArgs& a, cudaStream_t st);
int tc_launch_chunk_out(const ScanArgs& a, cudaStream_t st);
int tc_launch_chunk_dstate(const ScanArgs& a, cudaStream_t st);
int tc_launch_chunk_grads(const ScanArgs& a, cudaStream_t st);

static int check_common(const ScanArgs* a, int dtype, const char* who) {
  ORBIT_REQUIRE(a != nullptr, ERR_BAD_ARG, "%s: null argument block", who);
  ORBIT_REQUIRE(dtype == F32 || dtype == BF16, ERR_BAD_ARG, "%s: unknown dtype code %d", who, dtype);
  ORBIT_REQUIRE(a->B >= 0 && a->L >= 0 && a->H > 0 && a->R > 0 && a->O > 0 && a->G > 0 && a->N > 0, ERR_BAD_ARG,
                "%s: bad geometry B=%d L=%d H=%d R=%d O=%d G=%d N=%d", who, a->B, a->L, a->H, a->R, a->O, a->G, a->N);
  ORBIT_REQUIRE(a->R <= SCAN_MAX_RANK && a->O <= SCAN_MAX_RANK, ERR_UNSUPPORTED,
                "%s: ranks up to %d are served, got R=%d O=%d", who, SCAN_MAX_RANK, a->R, a->O);
  ORBIT_REQUIRE(a->T > 0 && a->nc == (a->L + a->T - 1) / a->T, ERR_BAD_ARG, "%s: nc=%d does not match L=%d, T=%d", who,
                a->nc, a->L, a->T);
  ORBIT_REQUIRE(a->u && a->Bhat && a->Chat && a->dA && a->w && a->wd && (a->Sin || a->Sin16) && a->atot, ERR_BAD_ARG,
                "%s: null u/Bhat/Chat/dA/w/wd/Sin/atot", who);
  return OK;
}

}  // namespace orbit

using namespace orbit;

extern "C" const char* orbit_last_error(void) { return g_err; }
extern "C" const char* orbit_version(void) { return "orbit_b200 0.1 (sm_100a)"; }
extern "C" int orbit_built_for_sm(void) { return 100; }

extern "C" int orbit_ssd_scan_pick_chunk(int R, int O, int G, int N, int precision, int backward, int limit) {
  if (precision == ORBIT_PRECISION_IO) return tc_pick_chunk(R, O, G, N, backward, limit);
  return gen_pick_chunk(R, O, G, N, backward, limit);
}

// One phase of the scan (see include/orbit_b200.h for the phase codes).
extern "C" int orbit_ssd_scan_phase(const orbit_scan_args* a, int phase, const float* state_in, float* state_out, int dtype,
                                    int precision, void* stream) {
  int rc = check_common(a, dtype, "orbit_ssd_scan_phase");
  if (rc != OK) return rc;
  ORBIT_REQUIRE(a->B > 0 && a->L > 0, ERR_BAD_ARG, "orbit_ssd_scan_phase: empty problem (B=%d, L=%d)", a->B, a->L);
  ORBIT_REQUIRE(precision == ORBIT_PRECISION_IEEE || precision == ORBIT_PRECISION_IO, ERR_BAD_ARG,
                "orbit_ssd_scan_phase: unknown precision code %d", precision);
  cudaStream_t st = (cudaStream_t)stream;
  const bool io = precision == ORBIT_PRECISION_IO;
  if (io) {
    const char* why = nullptr;
    if (!tc_supported(*a, dtype, &why)) return fail(ERR_UNSUPPORTED, "orbit_ssd_scan_phase: precision 'io' refused: %s", why);
  }
  if (phase >= ORBIT_PHASE_CHUNK_DSTATE && phase != ORBIT_PHASE_STATE_PASS_DRY) {
    ORBIT_REQUIRE(a->dy && a->dS, ERR_BAD_ARG, "orbit_ssd_scan_phase: null dy/dS");
  }
  switch (phase) {
    case ORBIT_PHASE_CHUNK_STATE: return io ? tc_launch_chunk_state(*a, st) : gen_launch_chunk_state(*a, dtype, st);
    case ORBIT_PHASE_STATE_PASS:
      ORBIT_REQUIRE(state_out != nullptr, ERR_BAD_ARG, "orbit_ssd_scan_phase: the forward pass needs state_out (S_fin)");
      return launch_state_pass_fwd(*a, state_in, state_out, st);
    case ORBIT_PHASE_CHUNK_OUT:
      ORBIT_REQUIRE(a->y != nullptr, ERR_BAD_ARG, "orbit_ssd_scan_phase: null y");
      return io ? tc_launch_chunk_out(*a, st) : gen_launch_chunk_out(*a, dtype, st);
    case ORBIT_PHASE_CHUNK_DSTATE: return io ? tc_launch_chunk_dstate(*a, st) : gen_launch_chunk_dstate(*a, dtype, st);
    case ORBIT_PHASE_STATE_PASS_BWD: return launch_state_pass_bwd(*a, state_in, state_out, st);
    case ORBIT_PHASE_STATE_PASS_DRY:
      ORBIT_REQUIRE(state_out != nullptr, ERR_BAD_ARG, "orbit_ssd_scan_phase: the dry pass needs state_out");
      return launch_state_pass_fwd(*a, state_in, state_out, st, true);
    case ORBIT_PHASE_STATE_PASS_BWD_DRY:
      ORBIT_REQUIRE(state_out != nullptr, ERR_BAD_ARG, "orbit_ssd_scan_phase: the dry reverse pass needs state_out");
      return launch_state_pass_bwd(*a, state_in, state_out, st, true);
    case ORBIT_PHASE_CHUNK_GRADS:
      ORBIT_REQUIRE(a->du && a->dBhat && a->dChat && a->ddA && a->dw, ERR_BAD_ARG,
                    "orbit_ssd_scan_phase: null du/dBhat/dChat/ddA/dw");
      return io ? tc_launch_chunk_grads(*a, st) : gen_launch_chunk_grads(*a, dtype, st);
    default: return fail(ERR_BAD_ARG, "orbit_ssd_scan_phase: unknown phase %d", phase);
  }
}

extern "C" int orbit_ssd_scan_fwd(const orbit_scan_args* a, const float* S0, float* S_fin, int dtype, int precision,
                                  void* stream) {
  int rc = check_common(a, dtype, "orbit_ssd_scan_fwd");
  if (rc != OK) return rc;
  ORBIT_REQUIRE(a->y && S_fin, ERR_BAD_ARG, "orbit_ssd_scan_fwd: null y/S_fin");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t state_elems = (int64_t)a->B * a->H * a->R * a->N * a->G;
  if (a->B == 0) return OK;
  if (a->L == 0) {   // nothing to scan: the state passes through
    if (S0) ORBIT_CHECK_CUDA(cudaMemcpyAsync(S_fin, S0, sizeof(float) * state_elems, cudaMemcpyDeviceToDevice, st));
    else ORBIT_CHECK_CUDA(cudaMemsetAsync(S_fin, 0, sizeof(float) * state_elems, st));
    return OK;
  }
  if (precision == ORBIT_PRECISION_IO) {
    const char* why = nullptr;
    if (!tc_supported(*a, dtype, &why)) return fail(ERR_UNSUPPORTED, "orbit_ssd_scan_fwd: precision 'io' refused: %s", why);
    if ((rc = tc_launch_chunk_state(*a, st)) != OK) return rc;
    if ((rc = launch_state_pass_fwd(*a, S0, S_fin, st)) != OK) return rc;
    return tc_launch_chunk_out(*a, st);
  }
  ORBIT_REQUIRE(precision == ORBIT_PRECISION_IEEE, ERR_BAD_ARG, "orbit_ssd_scan_fwd: unknown precision code %d", precision);
  if ((rc = gen_launch_chunk_state(*a, dtype, st)) != OK) return rc;
  if ((rc = launch_state_pass_fwd(*a, S0, S_fin, st)) != OK) return rc;
  return gen_launch_chunk_out(*a, dtype, st);
}

extern "C" int orbit_ssd_scan_bwd(const orbit_scan_args* a, const float* dS_fin, float* dS0, int dtype, int precision,
                                  void* stream) {
  int rc = check_common(a, dtype, "orbit_ssd_scan_bwd");
  if (rc != OK) return rc;
  ORBIT_REQUIRE(a->dy && a->du && a->dS && a->dBhat && a->dChat && a->ddA && a->dw, ERR_BAD_ARG,
                "orbit_ssd_scan_bwd: null dy/du/dS/dBhat/dChat/ddA/dw");
  ORBIT_REQUIRE((a->gBp == nullptr) == (a->dgBp == nullptr) && (a->gCp == nullptr) == (a->dgCp == nullptr) &&
                    (a->chi == nullptr) == (a->dchi == nullptr) && (a->beta == nullptr) == (a->dbeta_part == nullptr) &&
                    (a->gamma == nullptr) == (a->dgamma_part == nullptr) && (a->Dg == nullptr) == (a->dDg_part == nullptr),
                ERR_BAD_ARG, "orbit_ssd_scan_bwd: each optional operand needs its gradient buffer and vice versa");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t state_elems = (int64_t)a->B * a->H * a->R * a->N * a->G;
  if (a->B == 0) return OK;
  if (a->L == 0) {
    if (dS0) {
      if (dS_fin) ORBIT_CHECK_CUDA(cudaMemcpyAsync(dS0, dS_fin, sizeof(float) * state_elems, cudaMemcpyDeviceToDevice, st));
      else ORBIT_CHECK_CUDA(cudaMemsetAsync(dS0, 0, sizeof(float) * state_elems, st));
    }
    return OK;
  }
  if (precision == ORBIT_PRECISION_IO) {
    const char* why = nullptr;
    if (!tc_supported(*a, dtype, &why)) return fail(ERR_UNSUPPORTED, "orbit_ssd_scan_bwd: precision 'io' refused: %s", why);
    if ((rc = tc_launch_chunk_dstate(*a, st)) != OK) return rc;
    if ((rc = launch_state_pass_bwd(*a, dS_fin, dS0, st)) != OK) return rc;
    return tc_launch_chunk_grads(*a, st);
  }
  ORBIT_REQUIRE(precision == ORBIT_PRECISION_IEEE, ERR_BAD_ARG, "orbit_ssd_scan_bwd: unknown precision code %d", precision);
  if ((rc = gen_launch_chunk_dstate(*a, dtype, st)) != OK) return rc;
  if ((rc = launch_state_pass_bwd(*a, dS_fin, dS0, st)) != OK) return rc;
  return gen_launch_chunk_grads(*a, dtype, st);
}

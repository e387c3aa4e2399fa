/* orbit_b200: C-ABI of the B200 (sm_100a) kernels behind the `backend="cuda"` route of the SSD-MIMO layer.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (as void*), launches on that stream,
 * allocates nothing (workspaces are the caller's; sizes come from the *_workspace_bytes queries), never aborts or
 * traps, and returns an int status: 0 = ok, else one of ORBIT_ERR_* with the text available from
 * orbit_last_error() (thread-local).  dtype codes: 0 = float32, 1 = bfloat16 (the "IO dtype" of activations);
 * parameters, clocks, decays and states are always float32.
 *
 * Each declaration cites the interface of the reference project (d-rochau/OrbitSSM, paths inside that project)
 * that it stands in for.
 */
#ifndef ORBIT_B200_H
#define ORBIT_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ORBIT_OK 0
#define ORBIT_ERR_BAD_ARG 1
#define ORBIT_ERR_UNSUPPORTED 2
#define ORBIT_ERR_CUDA 3
#define ORBIT_ERR_WORKSPACE 4
#define ORBIT_ERR_DEVICE_TIMEOUT 5

#define ORBIT_F32 0
#define ORBIT_BF16 1

#define ORBIT_PRECISION_IEEE 0 /* fp32 operands on the FP32 pipe, any geometry          */
#define ORBIT_PRECISION_IO 1   /* bf16 operands on tcgen05 tensor cores, fp32 accumulate */

/* Text of the last failure reported on the calling thread ("" if none). */
const char* orbit_last_error(void);
/* Library version string, and the compute capability it was built for (100 = sm_100a). */
const char* orbit_version(void);
int orbit_built_for_sm(void);

/* ---- depthwise causal conv1d (+bias, +SiLU), token-major ------------------------------------------------------
 * Stands in for causal_conv1d_cl_fwd / causal_conv1d_cl_bwd (src/orbit_ssm/layers/conv.py:219-277) and their
 * Triton kernels (src/orbit_ssm/kernels/conv_triton.py:888, 924).
 *   x       [B, L, C] with element strides (x_batch_stride, x_row_stride, 1): a column slice of a wider buffer is fine
 *   weight  [C, W] fp32, bias [C] fp32 or NULL, W in 2..4
 *   window  [B, C, W] fp32 or NULL: the carried state; slots 1..W-1 are the raw inputs preceding x (NULL = zeros)
 *   y       [B, L, C] contiguous
 * Backward recomputes the pre-activation from x; dx may again be a strided slice; dwindow [B, C, W] fp32 or NULL
 * receives the gradient of the carried window; dweight [C, W] / dbias [C] are reduced in a fixed order
 * (bitwise reproducible) through `workspace`. */
int orbit_conv1d_fwd(const void* x, int64_t x_batch_stride, int64_t x_row_stride, const float* weight,
                     const float* bias, const float* window, void* y, int B, int L, int C, int W, int dtype,
                     int silu, void* stream);
int64_t orbit_conv1d_bwd_workspace_bytes(int B, int L, int C, int W);
int orbit_conv1d_bwd(const void* x, int64_t x_batch_stride, int64_t x_row_stride, const float* weight,
                     const float* bias, const float* window, const void* dy, void* dx, int64_t dx_batch_stride,
                     int64_t dx_row_stride, float* dwindow, float* dweight, float* dbias, void* workspace,
                     int64_t workspace_bytes, int B, int L, int C, int W, int dtype, int silu, void* stream);

/* ---- output gate + RMSNorm ------------------------------------------------------------------------------------
 * Stands in for gated_rms_norm (src/orbit_ssm/layers/norms.py:133-168; kernels src/orbit_ssm/kernels/gated_norm.py:
 * 30-128) and for the SwiGLU gate the layer applies after the scan (src/orbit_ssm/ssm/ssd_mimo_torch.py:619-622).
 *   out = rms_norm(y * silu(z)) * w        z == NULL: no gate;  w == NULL: no norm (then rstd may be NULL)
 *   y, out [M, D] contiguous; z [M, D] with row stride z_row_stride; w [D] fp32; rstd [M] fp32 (saved for backward)
 * Backward: dy [M, D] contiguous, dz with row stride dz_row_stride, dw [D] fp32 (fixed-order reduction). */
int orbit_gate_norm_fwd(const void* y, const void* z, int64_t z_row_stride, const float* w, void* out, float* rstd,
                        int64_t M, int D, float eps, int dtype, void* stream);
int64_t orbit_gate_norm_bwd_workspace_bytes(int64_t M, int D);
int orbit_gate_norm_bwd(const void* y, const void* z, int64_t z_row_stride, const float* w, const float* rstd,
                        const void* dout, void* dy, void* dz, int64_t dz_row_stride, float* dw, void* workspace,
                        int64_t workspace_bytes, int64_t M, int D, int dtype, void* stream);

/* Gate + RMSNorm backward for callers that cannot allocate device memory.  No counterpart in the reference.
 * Some hosts of this library never get to call cudaMalloc: a plugin loaded into a runtime that owns all device memory
 * and hands the plugin only its input and output pointers (a cgo / JNI / ctypes binding without an allocator of its
 * own), or a serving process whose device arena is carved up at start-up and closed afterwards, where a late
 * allocation would stall the device or simply fail.  For them this variant of orbit_gate_norm_bwd keeps the partial
 * sums of the weight gradient in a device array built into the library (9.25 MiB, held by every GPU that loads the
 * library until the process exits) instead of a caller workspace.  Arguments and results are those of
 * orbit_gate_norm_bwd without `workspace`.
 *   Limit: min(M, 592) * D <= 592 * 4096 floats (any M when D <= 4096); larger problems are refused with
 *          ORBIT_ERR_UNSUPPORTED and a message naming the sizes.  A gate-only call (w == NULL) has no weight gradient,
 *          uses no scratch and is served at any size.
 *   The array is per device and is looked up for the CURRENT device: the buffers must live on the current device
 *   (checked on `dy`; ORBIT_ERR_BAD_ARG otherwise).
 *   The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *   current) and remembers it; make that first call before any stream capture begins.
 *   It calls no cudaMalloc, cudaFree or other allocating routine.
 *   All calls on a device share the one array, which keeps whatever the last call left in it; nothing in it needs
 *   clearing between calls, but two calls that overlap on the GPU (different streams) race on it: serialise them. */
int orbit_gate_norm_bwd_noalloc(const void* y, const void* z, int64_t z_row_stride, const float* w, const float* rstd,
                                const void* dout, void* dy, void* dz, int64_t dz_row_stride, float* dw, int64_t M, int D,
                                int dtype, void* stream);

/* ---- SSD-MIMO chunked scan ------------------------------------------------------------------------------------
 * Stands in for ssd_mimo_scan (src/orbit_ssm/kernels/ssd_mimo/autograd.py:2247-2339) and its backward
 * (_SSDMimoFn.backward, same file :1462); the law is the chunked dual of src/orbit_ssm/ssm/ssd_mimo_torch.py:663-708.
 * Notation: B batch, L tokens, H heads, R/O input/output rank, G channels per head (P = G*R), N state rows,
 * T chunk length, nc = ceil(L/T).  Per kernel head (h, r) the maps are built in the kernel from head-shared ones:
 *   Bbar[s,q,:] = gBp[s,r,:] * Bhat[s,q,:] + beta[h,r,q,:]      Cbar[t,o,:] = gCp[t,o,:] * Chat[t,o,:] + gamma[h,r,o,:]
 *   y[t,g,o] = sum_r chi_r(t) ( sum_{s<=t,q} W_r[t,s] (Cbar[t,o,:].Bbar[s,q,:]) u[s,g,q] + a_r(t) Cbar[t,o,:].Sin_r[:,g]
 *                               + Dg[h,g,r,o] u[t,g,r] )
 *   W_r[t,s] = exp(cs_t - cs_s) w_s (s < t), wd_t (s = t);  cs = prefix sum of dA inside the chunk;  a_r = exp(cs)
 * All token-indexed tensors are token-major.  Optional pointers are NULL when the feature is off. */
typedef struct orbit_scan_args {
  int B, L, H, R, O, G, N;
  int T, nc;
  int hsplit;         /* 0 / 1: one CTA walks all heads of a (batch, chunk).  k > 1 (dividing H; rank-1 tensor-core
                         tiles only): k CTAs walk H/k heads each, and CHUNK_GRADS writes dBhat / dChat as k partial
                         buffers [k, B, L, R|O, N] that the caller sums                                       */
  const void* u;      /* [B, L, H, G, R]  drive, IO dtype                                            */
  const void* Bhat;   /* [B, L, R, N]     IO dtype, token stride b_ts elements                       */
  const void* gBp;    /* [B, L, R, N]     1 + gB, IO dtype, token stride gb_ts, or NULL              */
  const void* Chat;   /* [B, L, O, N]     IO dtype, token stride c_ts                                */
  const void* gCp;    /* [B, L, O, N]     1 + gC, IO dtype, token stride gc_ts, or NULL              */
  int64_t b_ts, gb_ts, c_ts, gc_ts;
  const float* beta;  /* [H, R, R, N]  (h, r, q, n) or NULL                                          */
  const float* gamma; /* [H, R, O, N]  or NULL                                                       */
  const float* chi;   /* [B, L, H, R]  sibling weights or NULL (= 1)                                 */
  const float* dA;    /* [B, L, H, R]  log decay                                                     */
  const float* w;     /* [B, L, H, R]  write weight of earlier tokens                                */
  const float* wd;    /* [B, L, H, R]  write weight of the own token (Euler: the same buffer as w)   */
  const float* Dg;    /* [H, G, R, O]  skip gains or NULL                                            */
  float* Sin;         /* [B, nc, H, R, N, G]  out: state entering each chunk (saved for backward)    */
  float* atot;        /* [B, nc, H, R]        out: chunk decay (saved for backward)                  */
  float* dS;          /* [B, nc, H, R, N, G]  backward scratch: gradient of the state leaving chunks */
  void* y;            /* [B, L, H, G, O]  out, IO dtype                                              */
  const void* dy;     /* [B, L, H, G, O]  IO dtype                                                   */
  void* du;           /* [B, L, H, G, R]  out, IO dtype                                              */
  float* dBhat;       /* [B, L, R, N]  out                                                           */
  float* dgBp;        /* [B, L, R, N]  out or NULL                                                   */
  float* dChat;       /* [B, L, O, N]  out                                                           */
  float* dgCp;        /* [B, L, O, N]  out or NULL                                                   */
  float* ddA;         /* [B, L, H, R]  out                                                           */
  float* dw;          /* [B, L, H, R]  out                                                           */
  float* dwd;         /* [B, L, H, R]  out or NULL (Euler: NULL, dw then holds both)                 */
  float* dchi;        /* [B, L, H, R]  out or NULL                                                   */
  float* dbeta_part;  /* [B*nc, H, R, R, N]  out: per-chunk partial sums, or NULL                    */
  float* dgamma_part; /* [B*nc, H, R, O, N]  out or NULL                                             */
  float* dDg_part;    /* [B*nc, H, G, R, O]  out or NULL                                             */
  int* status;        /* device int or NULL: set to 1 by a kernel whose bounded wait gave up         */
  void* Sin16;        /* [B, nc, H, R, N, G] bfloat16 state tiles written by the forward pass, or NULL; required (with
                         dS16 in backward) by precision "io" at rank 1 (R = O = 1), whose tiles read them by TMA.
                         There the pass writes ONLY these tiles: Sin keeps the chunk-local states of CHUNK_STATE and
                         may be NULL in the backward phases                                                       */
  void* dS16;         /* [B, nc, H, R, N, G] bfloat16 tiles of dS written by the reverse pass, or NULL (as Sin16)  */
  float* du32;        /* [B, L, H, G, R] fp32 scratch, or NULL; required by CHUNK_GRADS of precision "io" at rank 4
                         (R = O = 4), which sums the drive gradient of a head over its siblings there          */
} orbit_scan_args;

/* The scan runs as three chunk-parallel phases per direction (the decomposition of the reference's chunk-parallel
 * route, src/orbit_ssm/kernels/ssd_mimo/chunkpar.py:15-33); orbit_ssd_scan_fwd / _bwd run them in order, and
 * orbit_ssd_scan_phase runs one (for callers that time or overlap them):
 *   CHUNK_STATE     chunk-local states into a->Sin, chunk decays into a->atot
 *   STATE_PASS      serial walk over chunks: a->Sin becomes the state entering each chunk; state_in = S0 or NULL,
 *                   state_out = S_fin
 *   CHUNK_OUT       y
 *   CHUNK_DSTATE    adjoint chunk states into a->dS
 *   STATE_PASS_BWD  reverse walk: a->dS becomes the gradient of the state leaving each chunk; state_in = dS_fin or
 *                   NULL, state_out = dS0 or NULL
 *   CHUNK_GRADS     every other gradient
 *   STATE_PASS_DRY / STATE_PASS_BWD_DRY   the same walks without writing a->Sin / a->dS: only state_out is produced.
 *                   Context parallelism uses them: a rank first learns what its segment contributes to the state
 *                   (zero state_in), exchanges that with its peers, then runs the real walk from the true state. */
#define ORBIT_PHASE_CHUNK_STATE 0
#define ORBIT_PHASE_STATE_PASS 1
#define ORBIT_PHASE_CHUNK_OUT 2
#define ORBIT_PHASE_CHUNK_DSTATE 3
#define ORBIT_PHASE_STATE_PASS_BWD 4
#define ORBIT_PHASE_CHUNK_GRADS 5
#define ORBIT_PHASE_STATE_PASS_DRY 6
#define ORBIT_PHASE_STATE_PASS_BWD_DRY 7
int orbit_ssd_scan_phase(const orbit_scan_args* a, int phase, const float* state_in, float* state_out, int dtype,
                         int precision, void* stream);

/* Largest chunk length (a power of two, <= limit) whose working set fits one CTA for this geometry. */
int orbit_ssd_scan_pick_chunk(int R, int O, int G, int N, int precision, int backward, int limit);
/* Forward: S0 [B, H, R, N, G] fp32 or NULL (zero start); S_fin [B, H, R, N, G] fp32 out. */
int orbit_ssd_scan_fwd(const orbit_scan_args* a, const float* S0, float* S_fin, int dtype, int precision,
                       void* stream);
/* Backward: dS_fin [B, H, R, N, G] fp32 or NULL; dS0 [B, H, R, N, G] fp32 out or NULL.  Needs a->Sin and a->atot
 * as the forward left them. */
int orbit_ssd_scan_bwd(const orbit_scan_args* a, const float* dS_fin, float* dS0, int dtype, int precision,
                       void* stream);

/* One token (decode): the scan at L = 1 in one launch, any geometry the argument block can state; inference only.
 * Replaces the reference's `_step_core` inside `ssd_step` / `mixer_step_fast` (src/orbit_ssm/ssm/ssd_mimo_torch.py:388-490).
 * Reads u, the maps, clocks, chi, Dg of the block (all for the one token; a->L must be 1) and S0 [B, H, R, N, G] (NULL = zero);
 * writes a->y and the state after the token S1 (may alias S0: every element is read before it is written by its own thread). */
int orbit_ssd_scan_step(const orbit_scan_args* a, const float* S0, float* S1, int dtype, void* stream);

/* ---- token tails of the SSD-MIMO layer -------------------------------------------------------------------------
 * Replace the reference's `token_law` (src/orbit_ssm/ssm/ssd_mimo_torch.py:161-267; fused CUDA form `token_tails`,
 * src/orbit_ssm/layers/tails.py:829).  Slab columns are read in place (row strides in elements); gradients are written
 * in place into the gradient of the slab.
 *
 * Map tail: out[m, x, n] = (weight ? src[m, n*X + x] * rstd[m, x] * weight[n] : src[m, n*X + x]) + bias[n] + add, with
 * rstd[m, x] = rsqrt(mean_n src[m, n*X + x]^2 + eps)  (B / C maps: RMSNorm over the N state rows of each input / output
 * column; gates: weight = bias = NULL, add = 1).  src [M, N*X] IO dtype, out [M, X, N] IO dtype contiguous, rstd [M, X]. */
int orbit_token_map_fwd(const void* src, int64_t src_row_stride, const float* weight, const float* bias, float add, float eps,
                        void* out, float* rstd, int64_t M, int X, int N, int dtype, void* stream);
int64_t orbit_token_map_bwd_workspace_bytes(int N);
/* dsrc [M, N*X] (row stride dsrc_row_stride) receives the input gradient; dweight / dbias [N] (or NULL) the parameter
 * gradients (fixed-order two-stage sums through `workspace`). */
int orbit_token_map_bwd(const void* src, int64_t src_row_stride, const float* weight, const float* rstd, const void* dout,
                        void* dsrc, int64_t dsrc_row_stride, float* dweight, float* dbias, void* workspace,
                        int64_t workspace_bytes, int64_t M, int X, int N, int dtype, void* stream);

/* Clock tail: per (token, head, sibling)
 *   dt = softplus(dt_raw) (threshold 20);  rate = exp(A_log[h,r]) (a_act 0) | heavy tail (1) | softplus (2) of a_raw, floor 1e-4
 *   dA = -dt rate;  trapezoid (trap_raw != NULL): lam = sigmoid(trap_raw[h]), wd = lam dt, w_t = wd_t + dt_{t+1} (1 - lam_{t+1}),
 *   lag0 = dt_0 (1 - lam_0);  Euler: w = dt;  chi = r_mix[h,r] + rmix_raw.
 * Raw inputs are slab columns [M, .] in the IO dtype with their own row strides; outputs are fp32 [M, H, R]. */
typedef struct orbit_clock_args {
  int64_t M;                 /* rows = B * L                                                                       */
  int L, H, R;
  int a_act, a_per_sibling;  /* 0 static A_log; 1 heavy tail; 2 softplus.  a_raw is [M, H*R] if per sibling else [M, H]   */
  const void* dt_raw;   int64_t dt_rs;
  const void* a_raw;    int64_t a_rs;
  const void* trap_raw; int64_t trap_rs;      /* [M, H] or NULL (Euler)                                            */
  const void* rmix_raw; int64_t rmix_rs;      /* [M, H*R] or NULL                                                  */
  const float* A_log;        /* [H, R] or NULL                                                                     */
  const float* r_mix;        /* [H, R] or NULL (no chi)                                                            */
  float *dA, *w, *wd, *chi;  /* out [M, H, R]; wd only with a trapezoid, chi only with r_mix                       */
  float* lag0;               /* out [B, H, R] or NULL                                                              */
  /* backward */
  const float *ddA, *dw, *dwd, *dchi;   /* [M, H, R]; dwd / dchi may be NULL                                       */
  const float* dlag0;                   /* [B, H, R] or NULL                                                       */
  void* d_dt_raw;   int64_t ddt_rs;
  void* d_a_raw;    int64_t da_rs;
  void* d_trap_raw; int64_t dtrap_rs;
  void* d_rmix_raw; int64_t drmix_rs;
  float* g_alog;             /* out [M, H, R]: per-row term of dA_log (a_act 0); the caller sums it over rows      */
  /* optional: column sums over the rows of the UNROUNDED raw gradients = gradients of the slab biases, fp32, in the order
   * [ dt: H*R | a: H*R or H (a_act != 0) | trap: H (trapezoid) ]; fixed-order two-stage reduction                     */
  float* sum_part; int64_t sum_part_bytes;   /* workspace of orbit_token_clock_bwd_workspace_bytes(...) bytes, or NULL   */
  float* bias_sums;                          /* out [columns as above]; required with sum_part                           */
} orbit_clock_args;
int orbit_token_clock_fwd(const orbit_clock_args* a, int dtype, void* stream);
int64_t orbit_token_clock_bwd_workspace_bytes(int64_t M, int H, int R, int a_act, int a_per_sibling, int trap);
int orbit_token_clock_bwd(const orbit_clock_args* a, int dtype, void* stream);

/* ---- HybridMamba coordinate-decay scan -----------------------------------------------------------------------
 * Replaces the reference's `mh_scan` (src/orbit_ssm/kernels/hybrid_mamba_mh/functions.py:665-677; law restated from
 * src/orbit_ssm/kernels/hybrid_mamba_mh/torch_scan.py:44-76, 180-279) for `coord_static` rows, real and rotating:
 *   a_t[h,p,n] = exp(-exp(A_log[h,p,n]) delta_t[h])
 *   Theta_t[h,k] = Theta_{t-1}[h,k] + delta_t[h] feat_t[k]                       (pairs k with rot[k] != 0)
 *   Bt_t[h,:] = Rot(Theta_t)(Bh_t + beta_b[h]),  Ct_t[h,:] = Rot(Theta_t + theta_h[h])(Ch_t + beta_c[h])
 *   raw_t[p,n] = x_t[p] Bt_t[n];  h_t = a_t (h_{t-1} + delta_t (1 - lam_t) raw_{t-1}) + delta_t lam_t raw_t   (lam = 1: Euler)
 *   y_t[p] = sum_n Ct_t[n] h_t[p,n] + D[h] x_t[p]
 * Token-major tensors; the scan is sequential in time inside one CTA per (batch, head); the state entering every
 * chunk of `Tc` tokens (and the phase) is saved for the backward, which recomputes chunk interiors.
 * Envelope: P and N multiples of 4, N/4 a power of two <= 32, (P/4)(N/4) <= 256, Tc a multiple of 8 (32 for the backward). */
typedef struct orbit_hm_args {
  int B, L, H, P, N;
  int Tc, nck;              /* checkpoint interval in tokens, number of chunks = ceil(L / Tc)                   */
  const void* x;            /* [B, L, H*P]  IO dtype                                                            */
  const float* delta;       /* [B, L, H]    after softplus                                                      */
  const float* A_log;       /* [H, P, N]                                                                        */
  const float* Bh;          /* [B, L, N]    write map (after its norm)                                          */
  const float* Ch;          /* [B, L, N]    read map                                                            */
  const float* beta_b;      /* [H, N] or NULL                                                                   */
  const float* beta_c;      /* [H, N] or NULL                                                                   */
  const float* feat;        /* [B, L, N/2]  angle feature per pair, or NULL (no rotation)                       */
  const unsigned char* rot; /* [N/2]  1 = the pair rotates (required with feat)                                 */
  const float* theta_h;     /* [H, N/2] read offset in the scan's frame, or NULL                                */
  const float* lam;         /* [B, L, H] trapezoid weight, or NULL (Euler)                                      */
  const float* D;           /* [H] or NULL                                                                      */
  const float* h_init;      /* [B, H, P, N] or NULL                                                             */
  const float* write_prev;  /* [B, H, P, N] raw write of the token before the call, or NULL                     */
  const float* theta_init;  /* [B, H, N/2] or NULL                                                              */
  void* y;                  /* [B, L, H*P]  out, IO dtype                                                       */
  float* h_final;           /* [B, H, P, N] out                                                                 */
  float* theta_final;       /* [B, H, N/2]  out or NULL                                                         */
  float* write_last;        /* [B, H, P, N] out or NULL: raw write of the last token                            */
  float* hck;               /* [B, H, nck, P, N] out or NULL: state entering each chunk (saved for backward)    */
  float* thck;              /* [B, H, nck, N/2]  out or NULL: phase entering each chunk                         */
  /* backward only */
  const void* dy;           /* [B, L, H*P] IO dtype                                                             */
  const float* dh_final;    /* [B, H, P, N] or NULL                                                             */
  const float* dtheta_final;/* [B, H, N/2] or NULL                                                              */
  const float* dwrite_last; /* [B, H, P, N] or NULL                                                             */
  void* dx;                 /* [B, L, H*P] out, IO dtype                                                        */
  float* ddelta;            /* [B, L, H] out                                                                    */
  float* dlam;              /* [B, L, H] out or NULL                                                            */
  float* dA_log_part;       /* [B, H, P, N] out: per-batch partial sums                                         */
  float* dBh_part;          /* [H, B, L, N] out: per-head partial sums                                          */
  float* dCh_part;          /* [H, B, L, N] out                                                                 */
  float* dbeta_b_part;      /* [B, H, N] out or NULL                                                            */
  float* dbeta_c_part;      /* [B, H, N] out or NULL                                                            */
  float* dfeat_part;        /* [H, B, L, N/2] out or NULL                                                       */
  float* dtheta_h_part;     /* [B, H, N/2] out or NULL                                                          */
  float* dD_part;           /* [B, H] out or NULL                                                               */
  float* dh_init;           /* [B, H, P, N] out or NULL                                                         */
  float* dwrite_prev;       /* [B, H, P, N] out or NULL                                                         */
  float* dtheta_init;       /* [B, H, N/2] out or NULL                                                          */
} orbit_hm_args;

int orbit_hm_scan_fwd(const orbit_hm_args* a, int dtype, void* stream);
/* Needs hck / thck written by the forward with the same Tc.  Every partial-sum buffer is written in full (no
 * accumulation into caller memory, no atomics): the caller sums them over their leading axis. */
int orbit_hm_scan_bwd(const orbit_hm_args* a, int dtype, void* stream);

/* ---- HybridMamba clock tail ------------------------------------------------------------------------------------
 * Replaces the clock part of the reference's `_fused_hm_tails` (src/orbit_ssm/ssm/hybrid_mamba.py:1890-1931; `dt_softplus_cf`,
 * src/orbit_ssm/layers/tails.py:1086), its angle feature (`_theta_feature`, hybrid_mamba.py:971-1000) and the exact sigmoid of
 * the trapezoid weight (src/orbit_ssm/layers/layout.py:115-148).  Per row m = (batch, token):
 *   delta[m,h] = softplus(dt_raw[m,h] + dt_bias[h]) (threshold 20);  lam[m,h] = sigmoid(trap_raw[m,h] + trap_bias[h]);
 *   feat[m,k]  = omega[j] tanh(th_raw[m,j]) at k = rot_idx[j], 0 at the other row pairs.
 * Raw inputs are slab columns [M, .] in the IO dtype with their own row strides; outputs are fp32.  Backward writes the raw
 * gradients in the IO dtype (their own row strides) and the parameter-shaped gradients through `part` (two fixed-order stages). */
typedef struct orbit_hm_tail_args {
  int64_t M;                  /* rows = B * L                                                                       */
  int H, K, Krot;             /* heads; row pairs N / 2; rotating pairs                                             */
  const void* dt_raw;   int64_t dt_rs;        /* [M, H]                                                             */
  const void* trap_raw; int64_t trap_rs;      /* [M, H] or NULL (Euler write)                                       */
  const void* th_raw;   int64_t th_rs;        /* [M, Krot] or NULL (no rotating pairs)                              */
  const float* dt_bias;       /* [H]                                                                                */
  const float* trap_bias;     /* [H] or NULL                                                                        */
  const float* omega;         /* [Krot] angular rate of each rotating pair                                          */
  const int* rot_idx;         /* [Krot] row-pair index of each rotating pair, distinct, in [0, K)                   */
  float *delta, *lam, *feat;  /* out [M, H], [M, H], [M, K]; forward writes them, backward reads lam                */
  /* backward */
  const float *ddelta, *dlam, *dfeat;         /* [M, H], [M, H], [M, K]; each may be NULL (taken as zero)           */
  void* d_dt_raw;   int64_t d_dt_rs;
  void* d_trap_raw; int64_t d_trap_rs;
  void* d_th_raw;   int64_t d_th_rs;
  float *d_dt_bias, *d_trap_bias, *d_omega;   /* out [H], [H], [Krot]; each may be NULL                             */
  float* part; int64_t part_bytes;            /* workspace of orbit_hm_tail_bwd_workspace_bytes(M, H, Krot) bytes   */
} orbit_hm_tail_args;
int orbit_hm_tail_fwd(const orbit_hm_tail_args* a, int dtype, void* stream);
int64_t orbit_hm_tail_bwd_workspace_bytes(int64_t M, int H, int Krot);
int orbit_hm_tail_bwd(const orbit_hm_tail_args* a, int dtype, void* stream);

/* ---- context parallelism: the exchange step of the SSD-MIMO scan ------------------------------------------------
 * A sequence split over W ranks (rank j holds segment j) needs one all-gather per direction.  Rank j contributes the
 * record [ F_j | A_j ] (forward) or [ E_j | A_j | X_j ] (backward), all float32:
 *   F_j [B, H, R, N, G]  state its segment leaves when started from zero (ORBIT_PHASE_STATE_PASS_DRY writes it in place)
 *   A_j [B, H, R]        total log-decay of its segment (orbit_cp_state_pack sums dA over the segment into the record)
 *   E_j [B, H, R, N, G]  what its segment's outputs ask of the entering state (ORBIT_PHASE_STATE_PASS_BWD_DRY)
 *   X_j [B, H, R, N, G]  gradient a caller put on the state rank j returned (zeros if none)
 * orbit_cp_state_combine reads the W gathered records ([W][stride] floats, in this GPU's memory) and writes
 *   forward   S_r = sum_{j<r} exp(A_{j+1} + .. + A_{r-1}) F_j        the state entering this rank's segment
 *   backward  d_r: d_{W-1} = X_{W-1}, d_{j-1} = X_{j-1} + E_j + exp(A_j) d_j     gradient of the state leaving it.
 * n_state = B*H*R*N*G, per_head = N*G, BHR = B*H*R.  No counterpart in the reference, which is single-process; the terms
 * are those of its chunk-parallel pass (src/orbit_ssm/kernels/ssd_mimo/chunkpar.py:19-25) and of its State continuation
 * contract (src/orbit_ssm/ssm/ssd_mimo_torch.py:677-679). */
int64_t orbit_cp_record_floats(int64_t n_state, int BHR, int backward);
int64_t orbit_cp_state_pack_workspace_bytes(int B, int L, int HR);
/* workspace: slice sums of the two-stage (fixed-order) reduction over the segment, written in full before they are read. */
int orbit_cp_state_pack(const float* dA, float* record, int B, int L, int HR, int64_t n_state, void* workspace,
                        int64_t workspace_bytes, void* stream);
int orbit_cp_state_combine(const float* records, int64_t stride, int world, int rank, int64_t n_state, int per_head, int BHR,
                           int backward, float* out, void* stream);

/* ---- diagnostics ---------------------------------------------------------------------------------------------
 * One 128 x N x K tcgen05 tile through the same TMA boxes, shared-memory descriptors and TMEM read-out as the scan
 * kernels: D[128, N] fp32 = op(A) * op(B), A and B bfloat16.  mode bit 0: A given as [K, 128] (M contiguous) instead
 * of [128, K]; bit 1: B given as [K, N] instead of [N, K]; bit 2: A staged through registers with the manual swizzle;
 * bit 3: A staged in tensor memory (packed bfloat16 pairs) instead of shared memory.  K, N in {64, 128}.
 * *status (device int) becomes nonzero if a bounded device wait gave up.  No counterpart in the reference (its
 * kernels are Triton; there is no sm_100 path there). */
int orbit_selftest_umma(const void* A, const void* B, float* D, int mode, int K, int N, int* status, void* stream);

/* The wind-down of a bounded device-side wait, exercised without a fault: one CTA allocates tensor memory and waits at
 * most `polls` (1..4096) polls on a barrier that nothing arrives on; the wait gives up, *status (device int) is set to
 * 1, tensor memory is freed and the kernel returns.  A caller that reads *status == 1 maps it to
 * ORBIT_ERR_DEVICE_TIMEOUT.  No counterpart in the reference. */
int orbit_selftest_wait_timeout(int* status, int polls, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ORBIT_B200_H */

// SSD-MIMO chunked scan, precision "ieee": fp32 arithmetic on the FP32 pipe for any (R, O, G, N), forward and backward.
//
// Replaces, for fp32 operands, the reference's scan entry (src/orbit_ssm/kernels/ssd_mimo/autograd.py:2247) whose law is the
// chunked dual of src/orbit_ssm/ssm/ssd_mimo_torch.py:663-708.  The work is split in three chunk-parallel phases (the
// decomposition the reference uses inside one GPU, src/orbit_ssm/kernels/ssd_mimo/chunkpar.py:15-33):
//   state  : per (batch, chunk): chunk-local state  Z_r = sum_s e_r[s] Bbar_r[s]^T u[s],  chunk decay atot_r
//   pass   : per (batch, head, sibling): serial walk over chunks  Sin[c+1] = atot[c] Sin[c] + Z[c]    (scan_pass.cu)
//   output : per (batch, chunk): y = (sum_r chi_r W_r o (Cbar_r Bbar_r^T)) u + sum_r chi_r a_r Cbar_r Sin_r + skip
// and the backward mirrors them (adjoint chunk state, reverse pass, chunk gradients).  One CTA owns one (batch, chunk)
// and loops over heads and siblings, so every head-summed gradient (maps shared by all heads) is accumulated by its
// single owner in a fixed order: no atomics, bitwise reproducible.
//
// Per-kernel-head maps are formed in shared memory from the head-shared maps:
//   Bbar_r[s,q,n] = gBp[s,r,n] * Bhat[s,q,n] + beta[h,r,q,n]     Cbar_r[t,o,n] = gCp[t,o,n] * Chat[t,o,n] + gamma[h,r,o,n]
#include "common.cuh"
#include "../../include/orbit_b200.h"
#include "scan_args.h"

namespace orbit {

constexpr int GEN_THREADS = 256;

struct ChunkCtx {
  int b, c, t0, Tv;   // batch, chunk, first token, valid tokens in chunk
};

template <typename T>
__device__ __forceinline__ float ld_or(const T* p, int64_t i) { return ldf(p + i); }

// cs[t] = inclusive prefix of dA over the chunk (0 past the valid tokens), wv/wdv the write weights (0 past the end)
__device__ __forceinline__ void load_clock(const ScanArgs& a, const ChunkCtx& cx, int h, int r, float* cs, float* wv,
                                           float* wdv, float* chiv) {
  const int T = a.T;
  if (threadIdx.x < T) {
    int t = threadIdx.x;
    float d = 0.f, w = 0.f, wd = 0.f, ch = 1.f;
    if (t < cx.Tv) {
      int64_t i = (((int64_t)cx.b * a.L + cx.t0 + t) * a.H + h) * a.R + r;
      d = a.dA[i];
      w = a.w[i];
      wd = a.wd[i];
      if (a.chi) ch = a.chi[i];
    }
    cs[t] = d;
    wv[t] = w;
    wdv[t] = wd;
    chiv[t] = ch;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float acc = 0.f;
    for (int t = 0; t < T; ++t) { acc += cs[t]; cs[t] = acc; }
  }
  __syncthreads();
}

template <typename T>
__device__ __forceinline__ void build_bbar(const ScanArgs& a, const ChunkCtx& cx, int h, int r, float* Bbar) {
  const int Tn = a.T, R = a.R, N = a.N;
  const T* Bh = (const T*)a.Bhat;
  const T* gB = (const T*)a.gBp;
  for (int idx = threadIdx.x; idx < Tn * R * N; idx += GEN_THREADS) {
    int n = idx % N, q = (idx / N) % R, s = idx / (N * R);
    float v = 0.f;
    if (s < cx.Tv) {
      int64_t tok = (int64_t)cx.b * a.L + cx.t0 + s;
      v = ldf(Bh + tok * a.b_ts + q * N + n);
      if (gB) v *= ldf(gB + tok * a.gb_ts + r * N + n);
      if (a.beta) v += a.beta[(((int64_t)h * R + r) * R + q) * N + n];
    }
    Bbar[idx] = v;
  }
}

template <typename T>
__device__ __forceinline__ void build_cbar(const ScanArgs& a, const ChunkCtx& cx, int h, int r, float* Cbar) {
  const int Tn = a.T, O = a.O, N = a.N;
  const T* Ch = (const T*)a.Chat;
  const T* gC = (const T*)a.gCp;
  for (int idx = threadIdx.x; idx < Tn * O * N; idx += GEN_THREADS) {
    int n = idx % N, o = (idx / N) % O, t = idx / (N * O);
    float v = 0.f;
    if (t < cx.Tv) {
      int64_t tok = (int64_t)cx.b * a.L + cx.t0 + t;
      v = ldf(Ch + tok * a.c_ts + o * N + n);
      if (gC) v *= ldf(gC + tok * a.gc_ts + o * N + n);
      if (a.gamma) v += a.gamma[(((int64_t)h * a.R + r) * O + o) * N + n];
    }
    Cbar[idx] = v;
  }
}

// drive tile u[s][g][q] (channel h*P + g*R + q), zero past the valid tokens
template <typename T>
__device__ __forceinline__ void load_tile(const T* src, int64_t row_stride, const ChunkCtx& cx, int L, int Tn, int col0,
                                          int ncol, float* dst) {
  for (int idx = threadIdx.x; idx < Tn * ncol; idx += GEN_THREADS) {
    int j = idx % ncol, s = idx / ncol;
    dst[idx] = (s < cx.Tv) ? ldf(src + ((int64_t)cx.b * L + cx.t0 + s) * row_stride + col0 + j) : 0.f;
  }
}

__device__ __forceinline__ ChunkCtx make_ctx(const ScanArgs& a) {
  ChunkCtx cx;
  cx.c = blockIdx.x;
  cx.b = blockIdx.y;
  cx.t0 = cx.c * a.T;
  cx.Tv = min(a.T, a.L - cx.t0);
  return cx;
}

// ---------------------------------------------------------------------------------------------------
// forward: chunk state
// ---------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(GEN_THREADS) gen_chunk_state_kernel(ScanArgs a) {
  extern __shared__ float sm[];
  const int Tn = a.T, R = a.R, G = a.G, N = a.N, P = G * R;
  float* u = sm;                       // [T][G][R]
  float* Bbar = u + Tn * P;            // [T][R][N]
  float* cs = Bbar + Tn * R * N;       // [T] x4
  float *wv = cs + Tn, *wdv = wv + Tn, *chiv = wdv + Tn, *e = chiv + Tn;
  ChunkCtx cx = make_ctx(a);
  for (int h = 0; h < a.H; ++h) {
    __syncthreads();
    load_tile((const T*)a.u, (int64_t)a.H * P, cx, a.L, Tn, h * P, P, u);
    for (int r = 0; r < R; ++r) {
      load_clock(a, cx, h, r, cs, wv, wdv, chiv);
      if (threadIdx.x < Tn) e[threadIdx.x] = __expf(cs[Tn - 1] - cs[threadIdx.x]) * wv[threadIdx.x];
      build_bbar<T>(a, cx, h, r, Bbar);
      __syncthreads();
      float* Z = a.Sin + ((((int64_t)cx.b * a.nc + cx.c) * a.H + h) * R + r) * (int64_t)N * G;
      for (int idx = threadIdx.x; idx < N * G; idx += GEN_THREADS) {
        int g = idx % G, n = idx / G;
        float acc = 0.f;
        for (int s = 0; s < cx.Tv; ++s) {
          float dot = 0.f;
          for (int q = 0; q < R; ++q) dot = fmaf(Bbar[(s * R + q) * N + n], u[(s * G + g) * R + q], dot);
          acc = fmaf(e[s], dot, acc);
        }
        Z[idx] = acc;
      }
      if (threadIdx.x == 0) a.atot[(((int64_t)cx.b * a.nc + cx.c) * a.H + h) * R + r] = __expf(cs[Tn - 1]);
      __syncthreads();
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// forward: chunk output
// ---------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(GEN_THREADS) gen_chunk_out_kernel(ScanArgs a) {
  extern __shared__ float sm[];
  const int Tn = a.T, R = a.R, O = a.O, G = a.G, N = a.N, P = G * R;
  const int MS = O * Tn * R * Tn;
  float* u = sm;                       // [T][G][R]
  float* Bbar = u + Tn * P;            // [T][R][N]
  float* Cbar = Bbar + Tn * R * N;     // [T][O][N]
  float* Mh = Cbar + Tn * O * N;       // [t][o][s][q]
  float* yacc = Mh + MS;               // [T][G][O]
  float* cs = yacc + Tn * G * O;
  float *wv = cs + Tn, *wdv = wv + Tn, *chiv = wdv + Tn;
  ChunkCtx cx = make_ctx(a);
  for (int h = 0; h < a.H; ++h) {
    __syncthreads();
    load_tile((const T*)a.u, (int64_t)a.H * P, cx, a.L, Tn, h * P, P, u);
    for (int idx = threadIdx.x; idx < MS; idx += GEN_THREADS) Mh[idx] = 0.f;
    for (int idx = threadIdx.x; idx < Tn * G * O; idx += GEN_THREADS) yacc[idx] = 0.f;
    for (int r = 0; r < R; ++r) {
      load_clock(a, cx, h, r, cs, wv, wdv, chiv);
      build_bbar<T>(a, cx, h, r, Bbar);
      build_cbar<T>(a, cx, h, r, Cbar);
      __syncthreads();
      for (int idx = threadIdx.x; idx < MS; idx += GEN_THREADS) {
        int q = idx % R, s = (idx / R) % Tn, o = (idx / (R * Tn)) % O, t = idx / (R * Tn * O);
        if (s > t || t >= cx.Tv) continue;
        float wgt = (s == t) ? wdv[t] : __expf(cs[t] - cs[s]) * wv[s];
        const float* cp = Cbar + (t * O + o) * N;
        const float* bp = Bbar + (s * R + q) * N;
        float dot = 0.f;
        for (int n = 0; n < N; ++n) dot = fmaf(cp[n], bp[n], dot);
        Mh[idx] += chiv[t] * wgt * dot;
      }
      const float* Sin = a.Sin + ((((int64_t)cx.b * a.nc + cx.c) * a.H + h) * R + r) * (int64_t)N * G;
      for (int idx = threadIdx.x; idx < Tn * G * O; idx += GEN_THREADS) {
        int o = idx % O, g = (idx / O) % G, t = idx / (O * G);
        if (t >= cx.Tv) continue;
        const float* cp = Cbar + (t * O + o) * N;
        float dot = 0.f;
        for (int n = 0; n < N; ++n) dot = fmaf(cp[n], Sin[n * G + g], dot);
        yacc[idx] += chiv[t] * __expf(cs[t]) * dot;
        if (a.Dg) yacc[idx] += chiv[t] * a.Dg[(((int64_t)h * G + g) * R + r) * O + o] * u[(t * G + g) * R + r];
      }
      __syncthreads();
    }
    T* y = (T*)a.y;
    for (int idx = threadIdx.x; idx < Tn * G * O; idx += GEN_THREADS) {
      int o = idx % O, g = (idx / O) % G, t = idx / (O * G);
      if (t >= cx.Tv) continue;
      float acc = yacc[idx];
      for (int s = 0; s <= t; ++s)
        for (int q = 0; q < R; ++q) acc = fmaf(Mh[((t * O + o) * Tn + s) * R + q], u[(s * G + g) * R + q], acc);
      stf(y + (((int64_t)cx.b * a.L + cx.t0 + t) * a.H + h) * (int64_t)G * O + g * O + o, acc);
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// backward: adjoint chunk state  Gs_r[n,g] = sum_{t,o} chi_r(t) a_r(t) Cbar_r[t,o,n] dy[t,g,o]
// ---------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(GEN_THREADS) gen_chunk_dstate_kernel(ScanArgs a) {
  extern __shared__ float sm[];
  const int Tn = a.T, R = a.R, O = a.O, G = a.G, N = a.N;
  float* dy = sm;                      // [T][G][O]
  float* Cbar = dy + Tn * G * O;       // [T][O][N]
  float* cs = Cbar + Tn * O * N;
  float *wv = cs + Tn, *wdv = wv + Tn, *chiv = wdv + Tn, *f = chiv + Tn;
  ChunkCtx cx = make_ctx(a);
  for (int h = 0; h < a.H; ++h) {
    __syncthreads();
    load_tile((const T*)a.dy, (int64_t)a.H * G * O, cx, a.L, Tn, h * G * O, G * O, dy);
    for (int r = 0; r < R; ++r) {
      load_clock(a, cx, h, r, cs, wv, wdv, chiv);
      if (threadIdx.x < Tn) f[threadIdx.x] = chiv[threadIdx.x] * __expf(cs[threadIdx.x]);
      build_cbar<T>(a, cx, h, r, Cbar);
      __syncthreads();
      float* Gs = a.dS + ((((int64_t)cx.b * a.nc + cx.c) * a.H + h) * R + r) * (int64_t)N * G;
      for (int idx = threadIdx.x; idx < N * G; idx += GEN_THREADS) {
        int g = idx % G, n = idx / G;
        float acc = 0.f;
        for (int t = 0; t < cx.Tv; ++t) {
          float dot = 0.f;
          for (int o = 0; o < O; ++o) dot = fmaf(Cbar[(t * O + o) * N + n], dy[(t * G + g) * O + o], dot);
          acc = fmaf(f[t], dot, acc);
        }
        Gs[idx] = acc;
      }
      __syncthreads();
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// backward: chunk gradients.  a.dS holds dSout (gradient of the state LEAVING each chunk) after the reverse pass.
// ---------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(GEN_THREADS) gen_chunk_grads_kernel(ScanArgs a) {
  extern __shared__ float sm[];
  const int Tn = a.T, R = a.R, O = a.O, G = a.G, N = a.N, P = G * R;
  const int MS = O * Tn * R * Tn;
  float* u = sm;                       // [T][G][R]
  float* dy = u + Tn * P;              // [T][G][O]
  float* du = dy + Tn * G * O;         // [T][G][R]
  float* Bbar = du + Tn * P;           // [T][R][N]
  float* Cbar = Bbar + Tn * R * N;     // [T][O][N]
  float* dMh = Cbar + Tn * O * N;      // [t][o][s][q]
  float* Mh = dMh + MS;
  float* Sc = Mh + MS;                 // scores, then dSc in place
  float* Kts = Sc + MS;                // [T][T]
  float* cs = Kts + Tn * Tn;
  float *wv = cs + Tn, *wdv = wv + Tn, *chiv = wdv + Tn, *dcs = chiv + Tn, *dwv = dcs + Tn, *dwdv = dwv + Tn,
        *dchi = dwdv + Tn, *da = dchi + Tn, *de = da + Tn, *red = de + Tn;   // red: 32 floats
  ChunkCtx cx = make_ctx(a);
  const int64_t slot = (int64_t)cx.b * a.nc + cx.c;
  const T* Bh = (const T*)a.Bhat;
  const T* gB = (const T*)a.gBp;
  const T* Ch = (const T*)a.Chat;
  const T* gC = (const T*)a.gCp;

  for (int h = 0; h < a.H; ++h) {
    __syncthreads();
    load_tile((const T*)a.u, (int64_t)a.H * P, cx, a.L, Tn, h * P, P, u);
    load_tile((const T*)a.dy, (int64_t)a.H * G * O, cx, a.L, Tn, h * G * O, G * O, dy);
    for (int idx = threadIdx.x; idx < Tn * P; idx += GEN_THREADS) du[idx] = 0.f;
    __syncthreads();
    for (int idx = threadIdx.x; idx < MS; idx += GEN_THREADS) {
      int q = idx % R, s = (idx / R) % Tn, o = (idx / (R * Tn)) % O, t = idx / (R * Tn * O);
      float acc = 0.f;
      if (s <= t && t < cx.Tv)
        for (int g = 0; g < G; ++g) acc = fmaf(dy[(t * G + g) * O + o], u[(s * G + g) * R + q], acc);
      dMh[idx] = acc;
      Mh[idx] = 0.f;
    }
    for (int r = 0; r < R; ++r) {
      load_clock(a, cx, h, r, cs, wv, wdv, chiv);
      build_bbar<T>(a, cx, h, r, Bbar);
      build_cbar<T>(a, cx, h, r, Cbar);
      if (threadIdx.x < Tn) { dcs[threadIdx.x] = 0.f; dwv[threadIdx.x] = 0.f; dwdv[threadIdx.x] = 0.f; dchi[threadIdx.x] = 0.f; }
      __syncthreads();
      const int64_t so = ((slot * a.H + h) * R + r) * (int64_t)N * G;
      const float* Sin = a.Sin + so;
      const float* dSo = a.dS + so;
      const float atot = __expf(cs[Tn - 1]);
      // scores
      for (int idx = threadIdx.x; idx < MS; idx += GEN_THREADS) {
        int q = idx % R, s = (idx / R) % Tn, o = (idx / (R * Tn)) % O, t = idx / (R * Tn * O);
        float dot = 0.f;
        if (s <= t && t < cx.Tv) {
          const float* cp = Cbar + (t * O + o) * N;
          const float* bp = Bbar + (s * R + q) * N;
          for (int n = 0; n < N; ++n) dot = fmaf(cp[n], bp[n], dot);
        }
        Sc[idx] = dot;
      }
      __syncthreads();
      // K[t,s] = sum_{o,q} dMh o Sc ; per-row quantities
      for (int idx = threadIdx.x; idx < Tn * Tn; idx += GEN_THREADS) {
        int s = idx % Tn, t = idx / Tn;
        float acc = 0.f;
        if (s <= t && t < cx.Tv)
          for (int o = 0; o < O; ++o)
            for (int q = 0; q < R; ++q) {
              int i = ((t * O + o) * Tn + s) * R + q;
              acc = fmaf(dMh[i], Sc[i], acc);
            }
        Kts[idx] = acc;
      }
      // da[t] = sum_{o,g} dy[t,g,o] (Cbar[t,o,:] . Sin[:,g]);   de[s] = sum_{q,g} u[s,g,q] (Bbar[s,q,:] . dSo[:,g])
      for (int idx = threadIdx.x; idx < 2 * Tn; idx += GEN_THREADS) {
        int t = idx % Tn;
        float acc = 0.f;
        if (t < cx.Tv) {
          if (idx < Tn) {
            for (int o = 0; o < O; ++o)
              for (int g = 0; g < G; ++g) {
                float dot = 0.f;
                for (int n = 0; n < N; ++n) dot = fmaf(Cbar[(t * O + o) * N + n], Sin[n * G + g], dot);
                acc = fmaf(dy[(t * G + g) * O + o], dot, acc);
              }
          } else {
            for (int q = 0; q < R; ++q)
              for (int g = 0; g < G; ++g) {
                float dot = 0.f;
                for (int n = 0; n < N; ++n) dot = fmaf(Bbar[(t * R + q) * N + n], dSo[n * G + g], dot);
                acc = fmaf(u[(t * G + g) * R + q], dot, acc);
              }
          }
        }
        if (idx < Tn) da[t] = acc; else de[t] = acc;
      }
      __syncthreads();
      // Mh += chi W Sc ; Sc <- dSc = dMh chi W
      for (int idx = threadIdx.x; idx < MS; idx += GEN_THREADS) {
        int s = (idx / R) % Tn, t = idx / (R * Tn * O);
        float v = 0.f;
        if (s <= t && t < cx.Tv) {
          float wgt = (s == t) ? wdv[t] : __expf(cs[t] - cs[s]) * wv[s];
          float cw = chiv[t] * wgt;
          Mh[idx] += cw * Sc[idx];
          v = dMh[idx] * cw;
        }
        Sc[idx] = v;
      }
      // decay / weight / chi gradients from K, da, de (one thread per token: fixed order)
      if (threadIdx.x < Tn) {
        int t = threadIdx.x;
        float g_cs = 0.f, g_w = 0.f, g_chi = 0.f;
        if (t < cx.Tv) {
          for (int s = 0; s < t; ++s) {          // row sums (this token as t)
            float E = __expf(cs[t] - cs[s]);
            float lam = chiv[t] * Kts[t * Tn + s] * E * wv[s];
            g_cs += lam;
            g_chi = fmaf(E * wv[s], Kts[t * Tn + s], g_chi);
          }
          g_chi = fmaf(wdv[t], Kts[t * Tn + t], g_chi);
          for (int tt = t + 1; tt < cx.Tv; ++tt) {   // column sums (this token as s)
            float E = __expf(cs[tt] - cs[t]);
            float kk = chiv[tt] * Kts[tt * Tn + t] * E;
            g_cs -= kk * wv[t];
            g_w += kk;
          }
          float at = __expf(cs[t]);
          g_cs = fmaf(chiv[t] * at, da[t], g_cs);
          g_chi = fmaf(at, da[t], g_chi);
          float Et = __expf(cs[Tn - 1] - cs[t]);
          g_w = fmaf(Et, de[t], g_w);
          g_cs -= Et * wv[t] * de[t];
          if (a.Dg) {
            float sk = 0.f;
            for (int g = 0; g < G; ++g)
              for (int o = 0; o < O; ++o)
                sk = fmaf(dy[(t * G + g) * O + o] * a.Dg[(((int64_t)h * G + g) * R + r) * O + o], u[(t * G + g) * R + r], sk);
            g_chi += sk;
          }
          dwdv[t] = chiv[t] * Kts[t * Tn + t];
        }
        dcs[t] = g_cs;
        dwv[t] = g_w;
        dchi[t] = g_chi;
      }
      __syncthreads();
      // chunk-end terms: d cs[T-1] += sum_s e_s de_s + atot * <dSo, Sin>
      {
        float part = 0.f;
        for (int idx = threadIdx.x; idx < N * G; idx += GEN_THREADS) part = fmaf(dSo[idx], Sin[idx], part);
        float datot = block_sum(part, red);
        if (threadIdx.x == 0) {
          float acc = atot * datot;
          for (int s = 0; s < cx.Tv; ++s) acc = fmaf(__expf(cs[Tn - 1] - cs[s]) * wv[s], de[s], acc);
          dcs[Tn - 1] += acc;
          // d dA[k] = sum_{t >= k} d cs[t]
          float run = 0.f;
          for (int t = Tn - 1; t >= 0; --t) { run += dcs[t]; dcs[t] = run; }
        }
        __syncthreads();
      }
      if (threadIdx.x < cx.Tv) {
        int t = threadIdx.x;
        int64_t i = (((int64_t)cx.b * a.L + cx.t0 + t) * a.H + h) * R + r;
        a.ddA[i] = dcs[t];
        a.dw[i] = dwv[t];
        if (a.dwd) a.dwd[i] = dwdv[t];
        if (a.dchi) a.dchi[i] = dchi[t];
      }
      // dCbar[t,o,n] -> dChat, dgCp, dgamma
      {
        float* dgam = a.dgamma_part ? a.dgamma_part + ((slot * a.H + h) * R + r) * (int64_t)O * N : nullptr;
        for (int idx = threadIdx.x; idx < O * N; idx += GEN_THREADS) {
          int n = idx % N, o = idx / N;
          float gsum = 0.f;
          for (int t = 0; t < cx.Tv; ++t) {
            float acc = 0.f;
            for (int s = 0; s <= t; ++s)
              for (int q = 0; q < R; ++q) acc = fmaf(Sc[((t * O + o) * Tn + s) * R + q], Bbar[(s * R + q) * N + n], acc);
            float cr = 0.f;
            for (int g = 0; g < G; ++g) cr = fmaf(dy[(t * G + g) * O + o], Sin[n * G + g], cr);
            acc = fmaf(chiv[t] * __expf(cs[t]), cr, acc);
            gsum += acc;
            int64_t tok = (int64_t)cx.b * a.L + cx.t0 + t;
            float gc = gC ? ldf(gC + tok * a.gc_ts + o * N + n) : 1.f;
            float* dch = a.dChat + (tok * O + o) * N + n;
            bool first = (h == 0 && r == 0);
            *dch = (first ? 0.f : *dch) + acc * gc;
            if (a.dgCp) {
              float* dg = a.dgCp + (tok * O + o) * N + n;
              *dg = (first ? 0.f : *dg) + acc * ldf(Ch + tok * a.c_ts + o * N + n);
            }
          }
          if (dgam) dgam[idx] = gsum;
        }
      }
      // dBbar[s,q,n] -> dBhat, dgBp, dbeta   (one thread per state row n walks q, so the q-sum of dgBp stays in-thread)
      {
        float* dbet = a.dbeta_part ? a.dbeta_part + ((slot * a.H + h) * R + r) * (int64_t)R * N : nullptr;
        for (int n = threadIdx.x; n < N; n += GEN_THREADS) {
          float gsum[SCAN_MAX_RANK];
#pragma unroll
          for (int q = 0; q < SCAN_MAX_RANK; ++q) gsum[q] = 0.f;
          for (int s = 0; s < cx.Tv; ++s) {
            int64_t tok = (int64_t)cx.b * a.L + cx.t0 + s;
            float gb = gB ? ldf(gB + tok * a.gb_ts + r * N + n) : 1.f;
            float es = __expf(cs[Tn - 1] - cs[s]) * wv[s];
            float dgb = 0.f;
            for (int q = 0; q < R; ++q) {
              float acc = 0.f;
              for (int t = s; t < cx.Tv; ++t)
                for (int o = 0; o < O; ++o) acc = fmaf(Sc[((t * O + o) * Tn + s) * R + q], Cbar[(t * O + o) * N + n], acc);
              float cr = 0.f;
              for (int g = 0; g < G; ++g) cr = fmaf(u[(s * G + g) * R + q], dSo[n * G + g], cr);
              acc = fmaf(es, cr, acc);
              gsum[q] += acc;
              float* dbh = a.dBhat + (tok * R + q) * N + n;
              *dbh = ((h == 0 && r == 0) ? 0.f : *dbh) + acc * gb;
              dgb = fmaf(acc, ldf(Bh + tok * a.b_ts + q * N + n), dgb);
            }
            if (a.dgBp) {
              float* dg = a.dgBp + (tok * R + r) * N + n;
              *dg = (h == 0 ? 0.f : *dg) + dgb;
            }
          }
          if (dbet)
            for (int q = 0; q < R; ++q) dbet[q * N + n] = gsum[q];
        }
      }
      // du[s,g,q] += e_s sum_n Bbar[s,q,n] dSo[n,g]
      for (int idx = threadIdx.x; idx < Tn * P; idx += GEN_THREADS) {
        int q = idx % R, g = (idx / R) % G, s = idx / P;
        if (s >= cx.Tv) continue;
        float dot = 0.f;
        for (int n = 0; n < N; ++n) dot = fmaf(Bbar[(s * R + q) * N + n], dSo[n * G + g], dot);
        du[idx] = fmaf(__expf(cs[Tn - 1] - cs[s]) * wv[s], dot, du[idx]);
        if (a.Dg && q == r) {
          float sk = 0.f;
          for (int o = 0; o < O; ++o) sk = fmaf(a.Dg[(((int64_t)h * G + g) * R + r) * O + o], dy[(s * G + g) * O + o], sk);
          du[idx] = fmaf(chiv[s], sk, du[idx]);
        }
      }
      // dD partial [slot][h][g][r][o] = sum_t chi_r(t) dy[t,g,o] u[t,g,r]
      if (a.dDg_part) {
        float* dd = a.dDg_part + (slot * a.H + h) * (int64_t)G * R * O;
        for (int idx = threadIdx.x; idx < G * O; idx += GEN_THREADS) {
          int o = idx % O, g = idx / O;
          float acc = 0.f;
          for (int t = 0; t < cx.Tv; ++t) acc = fmaf(chiv[t] * dy[(t * G + g) * O + o], u[(t * G + g) * R + r], acc);
          dd[(g * R + r) * O + o] = acc;
        }
      }
      __syncthreads();
    }
    // du[s,g,q] += sum_{t>=s,o} Mh[t,o,s,q] dy[t,g,o]
    T* dup = (T*)a.du;
    for (int idx = threadIdx.x; idx < Tn * P; idx += GEN_THREADS) {
      int q = idx % R, g = (idx / R) % G, s = idx / P;
      if (s >= cx.Tv) continue;
      float acc = du[idx];
      for (int t = s; t < cx.Tv; ++t)
        for (int o = 0; o < O; ++o) acc = fmaf(Mh[((t * O + o) * Tn + s) * R + q], dy[(t * G + g) * O + o], acc);
      stf(dup + ((int64_t)cx.b * a.L + cx.t0 + s) * (int64_t)a.H * P + h * P + g * R + q, acc);
    }
  }
}


// ---------------------------------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------------------------------
static size_t gen_smem_state(const ScanArgs& a) { return sizeof(float) * ((size_t)a.T * a.G * a.R + (size_t)a.T * a.R * a.N + 5 * a.T); }
static size_t gen_smem_out(const ScanArgs& a) {
  size_t ms = (size_t)a.O * a.T * a.R * a.T;
  return sizeof(float) * ((size_t)a.T * a.G * a.R + (size_t)a.T * a.R * a.N + (size_t)a.T * a.O * a.N + ms + (size_t)a.T * a.G * a.O + 4 * a.T);
}
static size_t gen_smem_dstate(const ScanArgs& a) { return sizeof(float) * ((size_t)a.T * a.G * a.O + (size_t)a.T * a.O * a.N + 5 * a.T); }
static size_t gen_smem_grads(const ScanArgs& a) {
  size_t ms = (size_t)a.O * a.T * a.R * a.T;
  return sizeof(float) * (2 * (size_t)a.T * a.G * a.R + (size_t)a.T * a.G * a.O + (size_t)a.T * a.R * a.N + (size_t)a.T * a.O * a.N + 3 * ms +
                          (size_t)a.T * a.T + 10 * a.T + 32);
}
constexpr size_t GEN_SMEM_LIMIT = 200 * 1024;

int gen_pick_chunk(int R, int O, int G, int N, int backward, int limit) {
  ScanArgs a = {};
  a.R = R; a.O = O; a.G = G; a.N = N;
  int best = 1;
  for (int T = 1; T <= 64 && T <= limit; T *= 2) {
    a.T = T;
    size_t need = gen_smem_out(a);
    if (gen_smem_state(a) > need) need = gen_smem_state(a);
    if (backward) {
      if (gen_smem_grads(a) > need) need = gen_smem_grads(a);
      if (gen_smem_dstate(a) > need) need = gen_smem_dstate(a);
    }
    if (need <= GEN_SMEM_LIMIT) best = T;
  }
  return best;
}

template <typename K>
static int gen_launch(K kernel, const char* name, const ScanArgs& a, size_t smem, cudaStream_t st) {
  ORBIT_REQUIRE(a.T <= 64, ERR_UNSUPPORTED, "%s: chunk length %d exceeds 64", name, a.T);
  ORBIT_REQUIRE(smem <= GEN_SMEM_LIMIT, ERR_UNSUPPORTED, "%s: chunk length %d needs %zu bytes of shared memory (limit %zu); "
                "use orbit_ssd_scan_pick_chunk", name, a.T, smem, GEN_SMEM_LIMIT);
  ORBIT_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(a.nc, a.B);
  kernel<<<grid, GEN_THREADS, smem, st>>>(a);
  ORBIT_CHECK_LAUNCH(name);
  return OK;
}

int gen_launch_chunk_state(const ScanArgs& a, int dtype, cudaStream_t st) {
  if (dtype == BF16) return gen_launch(gen_chunk_state_kernel<__nv_bfloat16>, "gen_chunk_state_kernel", a, gen_smem_state(a), st);
  return gen_launch(gen_chunk_state_kernel<float>, "gen_chunk_state_kernel", a, gen_smem_state(a), st);
}
int gen_launch_chunk_out(const ScanArgs& a, int dtype, cudaStream_t st) {
  if (dtype == BF16) return gen_launch(gen_chunk_out_kernel<__nv_bfloat16>, "gen_chunk_out_kernel", a, gen_smem_out(a), st);
  return gen_launch(gen_chunk_out_kernel<float>, "gen_chunk_out_kernel", a, gen_smem_out(a), st);
}
int gen_launch_chunk_dstate(const ScanArgs& a, int dtype, cudaStream_t st) {
  if (dtype == BF16) return gen_launch(gen_chunk_dstate_kernel<__nv_bfloat16>, "gen_chunk_dstate_kernel", a, gen_smem_dstate(a), st);
  return gen_launch(gen_chunk_dstate_kernel<float>, "gen_chunk_dstate_kernel", a, gen_smem_dstate(a), st);
}
int gen_launch_chunk_grads(const ScanArgs& a, int dtype, cudaStream_t st) {
  if (dtype == BF16) return gen_launch(gen_chunk_grads_kernel<__nv_bfloat16>, "gen_chunk_grads_kernel", a, gen_smem_grads(a), st);
  return gen_launch(gen_chunk_grads_kernel<float>, "gen_chunk_grads_kernel", a, gen_smem_grads(a), st);
}

}  // namespace orbit

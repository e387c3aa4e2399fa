// HybridMamba coordinate-decay scan (per-(head, channel, row) decay, rotating row pairs, Euler / trapezoid write).
//
// Replaces the reference's mh_scan (src/orbit_ssm/kernels/hybrid_mamba_mh/functions.py:665; the law is restated from
// src/orbit_ssm/kernels/hybrid_mamba_mh/torch_scan.py:44-76, 180-279).  The recurrence has a different decay for every
// (p, n), so there is no contraction to put on the tensor cores: the work is one exp and a handful of FMAs per state
// element per token (MUFU / FP32 issue bound).  One CTA owns one (batch, head) and walks time; a thread owns a
// 4 (channels) x 4 (rows) tile of the state in registers.  Tokens are staged through shared memory in tiles of 8
// (drive, clocks, and the per-head maps: bias -> rotate by the running phase).  Reductions over rows (y, dx) are
// shuffles inside a group of N/4 lanes; reductions over channels (dB, dC) and over the whole state (ddelta, dlam) go
// through per-warp partials in shared memory that are summed in a fixed order: no atomics, bitwise reproducible.
//
// Backward: the forward saves the state entering every chunk of Tc = 32 tokens.  A chunk is first replayed to get the
// state entering each of its 8-token sub-chunks (kept in shared memory); then, last sub-chunk first, the sub-chunk is
// replayed with its 8 states held in registers and walked in reverse with the adjoint recurrence
//   G_t = Ct_t dy_t + a_{t+1} G_{t+1}.
#include "common.cuh"
#include "../../include/orbit_b200.h"

namespace orbit {

using HmArgs = ::orbit_hm_args;
constexpr int HM_TT = 8;        // tokens per tile
constexpr int HM_TC = 32;       // checkpoint interval the backward is written for
constexpr int HM_SUB = HM_TC / HM_TT;

struct HmGeo {
  int P, N, K, NG, active, nthr, nwarp;
};
__host__ __device__ inline HmGeo hm_geo(int P, int N) {
  HmGeo g;
  g.P = P; g.N = N; g.K = N / 2; g.NG = N / 4;
  g.active = (P / 4) * g.NG;
  g.nthr = (g.active + 31) / 32 * 32;
  g.nwarp = g.nthr / 32;
  return g;
}

// Shared-memory tile of 8 tokens (+ the token before them in row 0).
struct HmTile {
  float *xs, *dts, *lams, *Bt, *Ct, *cB, *sB, *cC, *sC, *dys, *thc;
};
__host__ __device__ inline size_t r4(size_t n) { return (n + 3) & ~(size_t)3; }
// Every array starts on a 16-byte boundary (xs, Bt, Ct, dys rows are read as float4).
__host__ __device__ inline size_t hm_tile_floats(const HmGeo& g, bool bwd) {
  size_t n = 9 * g.P + 9 * g.N + 9 * g.N + 12 + 12 + r4(g.K);
  if (bwd) n += 8 * g.P + 4 * r4(9 * g.K);
  return n;
}
__device__ inline float* hm_tile_carve(HmTile& t, float* p, const HmGeo& g, bool bwd) {
  t.xs = p; p += 9 * g.P;
  t.Bt = p; p += 9 * g.N;
  t.Ct = p; p += 9 * g.N;
  t.cB = t.sB = t.cC = t.sC = t.dys = nullptr;
  if (bwd) { t.dys = p; p += 8 * g.P; }
  t.dts = p; p += 12;
  t.lams = p; p += 12;
  t.thc = p; p += r4(g.K);
  if (bwd) {
    t.cB = p; p += r4(9 * g.K);
    t.sB = p; p += r4(9 * g.K);
    t.cC = p; p += r4(9 * g.K);
    t.sC = p; p += r4(9 * g.K);
  }
  return p;
}

// ---- raw staging of the next tile (cp.async, double-buffered): the global-memory latency of a tile is paid while the
// previous tile computes, not at the top of every tile.
struct HmRaw {
  unsigned char *x, *dy;     // [9][P], [8][P] in the IO dtype
  float *B, *C, *feat, *dt, *lam;   // [9][N], [9][N], [8][K], [9], [9]
};
__host__ __device__ inline size_t hm_raw_floats(const HmGeo& g) { return 9 * g.P + 8 * g.P + 2 * 9 * g.N + r4(8 * g.K) + 12 + 12; }
__device__ inline float* hm_raw_carve(HmRaw& r, float* p, const HmGeo& g) {
  r.x = reinterpret_cast<unsigned char*>(p); p += 9 * g.P;
  r.dy = reinterpret_cast<unsigned char*>(p); p += 8 * g.P;
  r.B = p; p += 9 * g.N;
  r.C = p; p += 9 * g.N;
  r.feat = p; p += r4(8 * g.K);
  r.dt = p; p += 12;
  r.lam = p; p += 12;
  return p;
}
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gsrc, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  const int sz = valid ? 4 : 0;                 // src-size 0: the 4 destination bytes are zero-filled
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(gsrc), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Issue the copies of tokens [t0 - 1, t0 + 8) (t0 < 0: nothing).  Tokens outside [0, L) are zero-filled.
template <typename T, bool BWD>
__device__ __forceinline__ void hm_prefetch(const HmArgs& a, const HmGeo& g, const HmRaw& rw, int b, int h, int t0) {
  if (t0 >= 0) {
    const int tid = threadIdx.x, nt = blockDim.x;
    constexpr int EPW = 4 / (int)sizeof(T);          // elements per 4-byte word
    const int wpr = g.P / EPW;                       // words per row
    const T* x = (const T*)a.x;
    for (int idx = tid; idx < 9 * wpr; idx += nt) {
      const int r = idx / wpr, w = idx % wpr, tok = t0 - 1 + r;
      const bool ok = tok >= 0 && tok < a.L;
      cp_async4(rw.x + (size_t)idx * 4, x + ((int64_t)b * a.L + (ok ? tok : 0)) * a.H * g.P + h * g.P + w * EPW, ok);
    }
    if (BWD) {
      const T* dy = (const T*)a.dy;
      for (int idx = tid; idx < 8 * wpr; idx += nt) {
        const int r = idx / wpr, w = idx % wpr, tok = t0 + r;
        const bool ok = tok < a.L;
        cp_async4(rw.dy + (size_t)idx * 4, dy + ((int64_t)b * a.L + (ok ? tok : 0)) * a.H * g.P + h * g.P + w * EPW, ok);
      }
    }
    for (int idx = tid; idx < 9 * g.N; idx += nt) {
      const int r = idx / g.N, n = idx % g.N, tok = t0 - 1 + r;
      const bool ok = tok >= 0 && tok < a.L;
      const int64_t o = ((int64_t)b * a.L + (ok ? tok : 0)) * g.N + n;
      cp_async4(rw.B + idx, a.Bh + o, ok);
      cp_async4(rw.C + idx, a.Ch + o, ok);
    }
    if (a.feat != nullptr)
      for (int idx = tid; idx < 8 * g.K; idx += nt) {
        const int r = idx / g.K, k = idx % g.K, tok = t0 + r;
        const bool ok = tok < a.L;
        cp_async4(rw.feat + idx, a.feat + ((int64_t)b * a.L + (ok ? tok : 0)) * g.K + k, ok);
      }
    if (tid < 9) {
      const int tok = t0 - 1 + tid;
      const bool ok = tok >= 0 && tok < a.L;
      const int64_t o = ((int64_t)b * a.L + (ok ? tok : 0)) * a.H + h;
      cp_async4(rw.dt + tid, a.delta + o, ok);
      if (a.lam != nullptr) cp_async4(rw.lam + tid, a.lam + o, ok);
    }
  }
  cp_async_commit();
}

// Build the tile of tokens [t0 - 1, t0 + 8) from its staged raw copy.  tile.thc holds the phase entering token t0 and
// leaves holding the phase after token t0 + 7.  Ends with a __syncthreads().
template <typename T, bool BWD>
__device__ __forceinline__ void hm_build_tile(const HmArgs& a, const HmGeo& g, HmTile& tl, const HmRaw& rw, int b, int h, int t0) {
  const int tid = threadIdx.x, nt = blockDim.x;
  cp_async_wait_all();
  __syncthreads();
  const T* rx = reinterpret_cast<const T*>(rw.x);
  for (int idx = tid; idx < 9 * g.P; idx += nt) tl.xs[idx] = ldf(rx + idx);
  if (BWD) {
    const T* rdy = reinterpret_cast<const T*>(rw.dy);
    for (int idx = tid; idx < 8 * g.P; idx += nt) tl.dys[idx] = ldf(rdy + idx);
  }
  if (tid < 9) {
    tl.dts[tid] = rw.dt[tid];
    tl.lams[tid] = a.lam ? rw.lam[tid] : 1.f;
  }
  // running phase per pair: row 0 (token t0 - 1) sees the entering phase, row r the phase after token t0 + r - 1
  float* ang = tl.Ct;   // rows of Ct are not yet written: borrow [9][K] of it for the angles
  if (a.feat != nullptr && tid < g.K) {
    float th = tl.thc[tid];
    ang[tid] = th;
#pragma unroll
    for (int r = 1; r < 9; ++r) {
      th = fmaf(rw.dt[r], rw.feat[(r - 1) * g.K + tid], th);       // zero-filled past the end of the sequence
      ang[r * g.K + tid] = th;
    }
    tl.thc[tid] = th;
  }
  __syncthreads();
  // maps: bias -> rotate.  The angles are read before Ct is overwritten (a pair's Ct entries sit at [r][2k], [r][2k+1],
  // its angle at [r][k]: a different thread's pair may own that slot), so stage the angles in registers first.
  const int npair = 9 * g.K;
  constexpr int MAXP = 20;
  float angs[MAXP];
  int cnt = 0;
  for (int idx = tid; idx < npair && cnt < MAXP; idx += nt) angs[cnt++] = a.feat ? ang[idx] : 0.f;
  __syncthreads();
  cnt = 0;
  for (int idx = tid; idx < npair && cnt < MAXP; idx += nt, ++cnt) {
    const int r = idx / g.K, k = idx % g.K, tok = t0 - 1 + r;
    float b0 = 0.f, b1 = 0.f, c0 = 0.f, c1 = 0.f;
    if (tok >= 0 && tok < a.L) {
      b0 = rw.B[r * g.N + 2 * k]; b1 = rw.B[r * g.N + 2 * k + 1]; c0 = rw.C[r * g.N + 2 * k]; c1 = rw.C[r * g.N + 2 * k + 1];
      if (a.beta_b) { b0 += a.beta_b[h * g.N + 2 * k]; b1 += a.beta_b[h * g.N + 2 * k + 1]; }
      if (a.beta_c) { c0 += a.beta_c[h * g.N + 2 * k]; c1 += a.beta_c[h * g.N + 2 * k + 1]; }
    }
    float cb = 1.f, sb = 0.f, cc = 1.f, sc = 0.f;
    if (a.feat != nullptr && a.rot[k]) {
      sincosf(angs[cnt], &sb, &cb);
      sincosf(a.theta_h ? angs[cnt] + a.theta_h[h * g.K + k] : angs[cnt], &sc, &cc);
    }
    tl.Bt[r * g.N + 2 * k] = b0 * cb - b1 * sb;
    tl.Bt[r * g.N + 2 * k + 1] = b0 * sb + b1 * cb;
    tl.Ct[r * g.N + 2 * k] = c0 * cc - c1 * sc;
    tl.Ct[r * g.N + 2 * k + 1] = c0 * sc + c1 * cc;
    if (BWD) { tl.cB[idx] = cb; tl.sB[idx] = sb; tl.cC[idx] = cc; tl.sC[idx] = sc; }
  }
  __syncthreads();
}

// sum over the NG consecutive lanes of a row group (NG a power of two <= 32)
__device__ __forceinline__ float group_sum(float v, int NG) {
  for (int o = NG >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// sum over the 32 / NG groups of a warp (lanes with equal lane % NG)
__device__ __forceinline__ float cross_group_sum(float v, int NG) {
  for (int o = NG; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sums 4 per-row partials over the NG lanes of a row group with a reduce-scatter (NG >= 4): 3 + log2(NG/4) shuffles
// instead of 4 log2(NG).  Every lane returns the total of row `row` (rows are dealt by two bits of the lane's position).
__device__ __forceinline__ float group_reduce4(const float (&v)[4], int NG, int ng, int& row) {
  const int hA = NG >> 1, hB = NG >> 2;
  const bool upA = (ng & hA) != 0, upB = (ng & hB) != 0;
  float k0 = upA ? v[2] : v[0], k1 = upA ? v[3] : v[1];
  const float s0 = upA ? v[0] : v[2], s1 = upA ? v[1] : v[3];
  k0 += __shfl_xor_sync(0xffffffffu, s0, hA);
  k1 += __shfl_xor_sync(0xffffffffu, s1, hA);
  float k = upB ? k1 : k0;
  const float s = upB ? k0 : k1;
  k += __shfl_xor_sync(0xffffffffu, s, hB);
  for (int o = hB >> 1; o > 0; o >>= 1) k += __shfl_xor_sync(0xffffffffu, k, o);
  row = (upA ? 2 : 0) + (upB ? 1 : 0);
  return k;
}
__device__ __forceinline__ float pick4(const float (&v)[4], int i) { return i == 0 ? v[0] : i == 1 ? v[1] : i == 2 ? v[2] : v[3]; }

struct HmThread {
  int pg, ng;        // channel group (4 channels), row group (4 rows)
  bool active;
};
__device__ __forceinline__ HmThread hm_thread(const HmGeo& g) {
  HmThread t;
  t.active = (int)threadIdx.x < g.active;
  const int id = t.active ? threadIdx.x : 0;
  t.pg = id / g.NG;
  t.ng = id % g.NG;
  return t;
}

constexpr float HM_LOG2E = 1.4426950408889634f, HM_LN2 = 0.6931471805599453f;
// 2^x on the MUFU pipe (one instruction; the decay exponents are <= 0, flush-to-zero of denormal results is harmless)
__device__ __forceinline__ float fast_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// one forward token on the thread's 4 x 4 tile.  rate2 = -exp(A_log) log2(e), so that a = 2^(rate2 delta).
template <bool TRAP>
__device__ __forceinline__ void hm_step(float (&hs)[16], float (&prv)[16], const float (&rate2)[16], const float4 x4,
                                        const float4 b4, float d, float lm) {
  const float xv[4] = {x4.x, x4.y, x4.z, x4.w}, bv[4] = {b4.x, b4.y, b4.z, b4.w};
  const float dl = d * lm, dg = d * (1.f - lm);
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int e = i * 4 + j;
      const float av = fast_ex2(rate2[e] * d);
      const float raw = xv[i] * bv[j];
      if (TRAP) hs[e] = fmaf(av, fmaf(dg, prv[e], hs[e]), dl * raw);
      else hs[e] = fmaf(av, hs[e], d * raw);
      prv[e] = raw;
    }
}

__device__ __forceinline__ void load16(float (&v)[16], const float* base, const HmThread& th, int N) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 r = *reinterpret_cast<const float4*>(base + (int64_t)(th.pg * 4 + i) * N + th.ng * 4);
    v[i * 4] = r.x; v[i * 4 + 1] = r.y; v[i * 4 + 2] = r.z; v[i * 4 + 3] = r.w;
  }
}
__device__ __forceinline__ void store16(const float (&v)[16], float* base, const HmThread& th, int N) {
#pragma unroll
  for (int i = 0; i < 4; ++i)
    *reinterpret_cast<float4*>(base + (int64_t)(th.pg * 4 + i) * N + th.ng * 4) = make_float4(v[i * 4], v[i * 4 + 1], v[i * 4 + 2], v[i * 4 + 3]);
}

// ---------------------------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------------------------
template <typename T, bool TRAP>
__global__ void __launch_bounds__(256) hm_fwd_kernel(const HmArgs a) {
  extern __shared__ __align__(16) float smf[];
  const HmGeo g = hm_geo(a.P, a.N);
  HmTile tl;
  float* ys = hm_tile_carve(tl, smf, g, false);      // [8][P]
  HmRaw raw[2];
  float* rp = hm_raw_carve(raw[0], ys + 8 * g.P, g);
  hm_raw_carve(raw[1], rp, g);
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
  hm_prefetch<T, false>(a, g, raw[0], b, h, 0);
  const HmThread th = hm_thread(g);
  constexpr bool trap = TRAP;
  const int64_t bh = (int64_t)b * a.H + h;
  float hs[16], prv[16], rate[16];
  load16(rate, a.A_log + (int64_t)h * g.P * g.N, th, g.N);
#pragma unroll
  for (int e = 0; e < 16; ++e) { rate[e] = -__expf(rate[e]) * HM_LOG2E; hs[e] = 0.f; prv[e] = 0.f; }
  if (a.h_init) load16(hs, a.h_init + bh * g.P * g.N, th, g.N);
  if (a.write_prev && trap) load16(prv, a.write_prev + bh * g.P * g.N, th, g.N);
  if (tid < g.K) tl.thc[tid] = a.theta_init ? a.theta_init[bh * g.K + tid] : 0.f;
  const float Dh = a.D ? a.D[h] : 0.f;
  __syncthreads();
  T* y = (T*)a.y;
  for (int t0 = 0; t0 < a.L; t0 += HM_TT) {
    if (a.hck != nullptr && t0 % a.Tc == 0) {
      const int c = t0 / a.Tc;
      if (th.active) store16(hs, a.hck + (bh * a.nck + c) * g.P * g.N, th, g.N);
      if (a.thck != nullptr && tid < g.K) a.thck[(bh * a.nck + c) * g.K + tid] = tl.thc[tid];
    }
    const int it = t0 / HM_TT;
    hm_build_tile<T, false>(a, g, tl, raw[it & 1], b, h, t0);
    hm_prefetch<T, false>(a, g, raw[(it + 1) & 1], b, h, t0 + HM_TT < a.L ? t0 + HM_TT : -1);
    const int nv = min(HM_TT, a.L - t0);
#pragma unroll
    for (int tt = 0; tt < HM_TT; ++tt) {
      if (tt < nv) {
        const float4 x4 = *reinterpret_cast<const float4*>(tl.xs + (tt + 1) * g.P + th.pg * 4);
        const float4 b4 = *reinterpret_cast<const float4*>(tl.Bt + (tt + 1) * g.N + th.ng * 4);
        const float4 c4 = *reinterpret_cast<const float4*>(tl.Ct + (tt + 1) * g.N + th.ng * 4);
        hm_step<TRAP>(hs, prv, rate, x4, b4, tl.dts[tt + 1], tl.lams[tt + 1]);
        const float cv[4] = {c4.x, c4.y, c4.z, c4.w}, xv[4] = {x4.x, x4.y, x4.z, x4.w};
        float yp[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          yp[i] = 0.f;
#pragma unroll
          for (int j = 0; j < 4; ++j) yp[i] = fmaf(cv[j], hs[i * 4 + j], yp[i]);
        }
        if (g.NG >= 4) {
          int row;
          const float tot = group_reduce4(yp, g.NG, th.ng, row);
          if (th.active && (th.ng & ((g.NG >> 2) - 1)) == 0) ys[tt * g.P + th.pg * 4 + row] = fmaf(Dh, pick4(xv, row), tot);
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float tot = group_sum(yp[i], g.NG);
            if (th.active && th.ng == 0) ys[tt * g.P + th.pg * 4 + i] = fmaf(Dh, xv[i], tot);
          }
        }
      }
    }
    __syncthreads();
    for (int idx = tid; idx < nv * g.P; idx += blockDim.x) {
      const int tt = idx / g.P, p = idx % g.P;
      stf(y + ((int64_t)b * a.L + t0 + tt) * a.H * g.P + h * g.P + p, ys[idx]);
    }
    // the next tile's builder starts with writes to xs (not ys) and syncs before anything reads ys again
  }
  if (th.active) {
    store16(hs, a.h_final + bh * g.P * g.N, th, g.N);
    if (a.write_last) store16(prv, a.write_last + bh * g.P * g.N, th, g.N);
  }
  if (a.theta_final != nullptr && tid < g.K) a.theta_final[bh * g.K + tid] = tl.thc[tid];
}

// ---------------------------------------------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------------------------------------------
template <typename T, bool TRAP>
__global__ void __launch_bounds__(256, 1) hm_bwd_kernel(const HmArgs a) {
  extern __shared__ __align__(16) float smf[];
  const HmGeo g = hm_geo(a.P, a.N);
  HmTile tl;
  float* p = hm_tile_carve(tl, smf, g, true);
  float* hsub = p;  p += (size_t)HM_SUB * g.P * g.N;     // state entering each sub-chunk of the current chunk
  float* thsub = p; p += r4(HM_SUB * g.K);               // phase entering each sub-chunk
  float* partB = p; p += 8 * g.nwarp * g.N;              // [tt][warp][n]
  float* partC = p; p += 8 * g.nwarp * g.N;
  float* partS = p; p += 8 * g.nwarp * 2;                // [tt][warp][ddelta, dlam]
  float* dxs = p;   p += 8 * g.P;
  float* phs = p;   p += 8 * g.K;                        // [tt][k] feat * suffix (phase part of ddelta)
  float* Ssuf = p;  p += r4(g.K);                          // suffix sum of dTheta carried backwards in time
  float* red = p;   p += 32;
  HmRaw raw[2];
  p = hm_raw_carve(raw[0], p, g);
  p = hm_raw_carve(raw[1], p, g);
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // The tiles are visited in a fixed order: per chunk (last first) the first nsub - 1 sub-chunks forwards (replay), then
  // all nsub sub-chunks backwards.  item_t0(c, k) = first token of the k-th visit of chunk c, continuing into chunk c - 1.
  auto n_sub = [&](int c) { return min(HM_SUB, (a.L - c * HM_TC + HM_TT - 1) / HM_TT); };
  auto item_t0 = [&](int c, int k) -> int {
    int ns = n_sub(c);
    if (k >= 2 * ns - 1) {
      c -= 1;
      k = 0;
      if (c < 0) return -1;
      ns = HM_SUB;
    }
    return c * HM_TC + (k < ns - 1 ? k : (ns - 1) - (k - (ns - 1))) * HM_TT;
  };
  int seq = 0;
  hm_prefetch<T, true>(a, g, raw[0], b, h, item_t0(a.nck - 1, 0));
  const HmThread th = hm_thread(g);
  constexpr bool trap = TRAP;
  const int64_t bh = (int64_t)b * a.H + h;
  const int64_t PN = (int64_t)g.P * g.N;
  float rate[16], G[16], dA[16];
  load16(rate, a.A_log + (int64_t)h * PN, th, g.N);
#pragma unroll
  for (int e = 0; e < 16; ++e) { rate[e] = -__expf(rate[e]) * HM_LOG2E; G[e] = 0.f; dA[e] = 0.f; }
  if (a.dh_final) load16(G, a.dh_final + bh * PN, th, g.N);
  if (tid < g.K) Ssuf[tid] = a.dtheta_final ? a.dtheta_final[bh * g.K + tid] : 0.f;
  float lagn = 0.f;                       // delta_{t+1} (1 - lam_{t+1}) of the token processed just before (in reverse)
  float acc_bb = 0.f, acc_bc = 0.f;       // thread n < N: dbeta_b[n], dbeta_c[n]
  float acc_th = 0.f;                     // thread k < K: dtheta_h[k]
  float acc_D = 0.f;                      // thread p < P: partial of dD
  const float Dh = a.D ? a.D[h] : 0.f;
  T* dx = (T*)a.dx;
  __syncthreads();

  for (int c = a.nck - 1; c >= 0; --c) {
    const int tc0 = c * HM_TC;
    int item = 0;
    // ---- replay the chunk once, keeping the state and phase that enter each sub-chunk
    {
      float hs[16], prv[16];
      load16(hs, a.hck + (bh * a.nck + c) * PN, th, g.N);
      if (tid < g.K) tl.thc[tid] = a.thck ? a.thck[(bh * a.nck + c) * g.K + tid] : 0.f;
      __syncthreads();
      for (int j = 0; j < HM_SUB; ++j) {
        const int t0 = tc0 + j * HM_TT;
        if (t0 >= a.L) break;
        if (th.active) store16(hs, hsub + (size_t)j * PN, th, g.N);
        if (tid < g.K) thsub[j * g.K + tid] = tl.thc[tid];
        if (j == n_sub(c) - 1) break;      // the last sub-chunk is replayed below anyway
        hm_build_tile<T, false>(a, g, tl, raw[seq & 1], b, h, t0);
        ++item;
        ++seq;
        hm_prefetch<T, true>(a, g, raw[seq & 1], b, h, item_t0(c, item));
        if (j == 0) {
#pragma unroll
          for (int e = 0; e < 16; ++e) prv[e] = 0.f;
          if (trap) {
            if (t0 == 0) {
              if (a.write_prev) load16(prv, a.write_prev + bh * PN, th, g.N);
            } else {
              const float4 x4 = *reinterpret_cast<const float4*>(tl.xs + th.pg * 4);
              const float4 b4 = *reinterpret_cast<const float4*>(tl.Bt + th.ng * 4);
              const float xv[4] = {x4.x, x4.y, x4.z, x4.w}, bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
              for (int e = 0; e < 16; ++e) prv[e] = xv[e >> 2] * bv[e & 3];
            }
          }
        }
        const int nv = min(HM_TT, a.L - t0);
        for (int tt = 0; tt < nv; ++tt) {
          const float4 x4 = *reinterpret_cast<const float4*>(tl.xs + (tt + 1) * g.P + th.pg * 4);
          const float4 b4 = *reinterpret_cast<const float4*>(tl.Bt + (tt + 1) * g.N + th.ng * 4);
          hm_step<TRAP>(hs, prv, rate, x4, b4, tl.dts[tt + 1], tl.lams[tt + 1]);
        }
        __syncthreads();
      }
      __syncthreads();
    }
    // ---- sub-chunks, last first
    for (int j = HM_SUB - 1; j >= 0; --j) {
      const int t0 = tc0 + j * HM_TT;
      if (t0 >= a.L) continue;
      if (tid < g.K) tl.thc[tid] = thsub[j * g.K + tid];
      __syncthreads();
      hm_build_tile<T, true>(a, g, tl, raw[seq & 1], b, h, t0);
      ++item;
      ++seq;
      hm_prefetch<T, true>(a, g, raw[seq & 1], b, h, item_t0(c, item));
      // The sub-chunk is walked in two halves of 4 tokens (second half first): a half's 4 states are held in registers;
      // the first half is replayed once more from the sub-chunk boundary.  (Keeping all 8 states costs 128 registers
      // and an unrolled body that no longer fits the instruction cache.)
      float hist[4][16];
#pragma unroll 1
      for (int half = 1; half >= 0; --half) {
      float prv0[16];                            // raw write of the token before token 4 * half
      {
        float hs[16], prv[16];
        load16(hs, hsub + (size_t)j * PN, th, g.N);
#pragma unroll
        for (int e = 0; e < 16; ++e) prv[e] = 0.f;
        if (trap) {
          if (t0 == 0) {
            if (a.write_prev) load16(prv, a.write_prev + bh * PN, th, g.N);
          } else {
            const float4 x4 = *reinterpret_cast<const float4*>(tl.xs + th.pg * 4);
            const float4 b4 = *reinterpret_cast<const float4*>(tl.Bt + th.ng * 4);
            const float xv[4] = {x4.x, x4.y, x4.z, x4.w}, bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
            for (int e = 0; e < 16; ++e) prv[e] = xv[e >> 2] * bv[e & 3];
          }
        }
        if (half == 1) {
#pragma unroll
          for (int tt = 0; tt < 4; ++tt) {
            const float4 x4 = *reinterpret_cast<const float4*>(tl.xs + (tt + 1) * g.P + th.pg * 4);
            const float4 b4 = *reinterpret_cast<const float4*>(tl.Bt + (tt + 1) * g.N + th.ng * 4);
            hm_step<TRAP>(hs, prv, rate, x4, b4, tl.dts[tt + 1], tl.lams[tt + 1]);
          }
        }
#pragma unroll
        for (int e = 0; e < 16; ++e) prv0[e] = prv[e];
#pragma unroll
        for (int k = 0; k < 4; ++k) {              // tokens past L: zero clock and drive leave the state unchanged
          const int tt = half * 4 + k;
          const float4 x4 = *reinterpret_cast<const float4*>(tl.xs + (tt + 1) * g.P + th.pg * 4);
          const float4 b4 = *reinterpret_cast<const float4*>(tl.Bt + (tt + 1) * g.N + th.ng * 4);
          hm_step<TRAP>(hs, prv, rate, x4, b4, tl.dts[tt + 1], tl.lams[tt + 1]);
#pragma unroll
          for (int e = 0; e < 16; ++e) hist[k][e] = hs[e];
        }
      }
      // ---- reverse walk
#pragma unroll
      for (int k = 3; k >= 0; --k) {
        const int tt = half * 4 + k;
        const int tok = t0 + tt;
        const float d = tl.dts[tt + 1], lm = tl.lams[tt + 1];
        const float4 x4 = *reinterpret_cast<const float4*>(tl.xs + (tt + 1) * g.P + th.pg * 4);
        const float4 xp4 = *reinterpret_cast<const float4*>(tl.xs + tt * g.P + th.pg * 4);
        const float4 b4 = *reinterpret_cast<const float4*>(tl.Bt + (tt + 1) * g.N + th.ng * 4);
        const float4 bp4 = *reinterpret_cast<const float4*>(tl.Bt + tt * g.N + th.ng * 4);
        const float4 c4 = *reinterpret_cast<const float4*>(tl.Ct + (tt + 1) * g.N + th.ng * 4);
        const float4 dy4 = *reinterpret_cast<const float4*>(tl.dys + tt * g.P + th.pg * 4);
        const float xv[4] = {x4.x, x4.y, x4.z, x4.w}, xpv[4] = {xp4.x, xp4.y, xp4.z, xp4.w};
        const float bv[4] = {b4.x, b4.y, b4.z, b4.w}, bpv[4] = {bp4.x, bp4.y, bp4.z, bp4.w};
        const float cv[4] = {c4.x, c4.y, c4.z, c4.w}, dyv[4] = {dy4.x, dy4.y, dy4.z, dy4.w};
        float px[4] = {0.f, 0.f, 0.f, 0.f}, pB[4] = {0.f, 0.f, 0.f, 0.f}, pC[4] = {0.f, 0.f, 0.f, 0.f};
        float sQ = 0.f, S1 = 0.f, S2 = 0.f;        // sums of dlog rate2, G raw, (a G) raw_prev over this thread's tile
        const float dl = d * lm, dg = d * (1.f - lm);
        const bool last = (tok == a.L - 1) && a.dwrite_last != nullptr;
        if (tok < a.L) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int jn = 0; jn < 4; ++jn) {
              const int e = i * 4 + jn;
              const float Gt = fmaf(cv[jn], dyv[i], G[e]);
              pC[jn] = fmaf(dyv[i], hist[k][e], pC[jn]);
              const float raw = xv[i] * bv[jn];
              const float u1 = Gt * raw;
              const float q = fmaf(Gt, hist[k][e], -dl * u1) * rate[e];   // dL / d log a_t, times rate2
              dA[e] = fmaf(q, d, dA[e]);
              sQ += q;
              const float aG = fast_ex2(rate[e] * d) * Gt;
              float draw = fmaf(dl, Gt, lagn * G[e]);
              if (last) draw += a.dwrite_last[bh * PN + (int64_t)(th.pg * 4 + i) * g.N + th.ng * 4 + jn];
              S1 += u1;
              if (TRAP) {
                const float rawp = (k == 0) ? prv0[e] : xpv[i] * bpv[jn];
                S2 = fmaf(aG, rawp, S2);
              }
              px[i] = fmaf(draw, bv[jn], px[i]);
              pB[jn] = fmaf(draw, xv[i], pB[jn]);
              G[e] = aG;
            }
          lagn = dg;
        }
        float sD = fmaf(HM_LN2, sQ, fmaf(lm, S1, (1.f - lm) * S2)), sL = d * (S1 - S2);
        if (!th.active) { sD = 0.f; sL = 0.f; }
        if (g.NG >= 4) {
          int row;
          const float tot = group_reduce4(px, g.NG, th.ng, row);
          if (th.active && (th.ng & ((g.NG >> 2) - 1)) == 0) dxs[tt * g.P + th.pg * 4 + row] = fmaf(Dh, pick4(dyv, row), tot);
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float v = group_sum(px[i], g.NG);
            if (th.active && th.ng == 0) dxs[tt * g.P + th.pg * 4 + i] = fmaf(Dh, dyv[i], v);
          }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float vb = th.active ? pB[i] : 0.f, vc = th.active ? pC[i] : 0.f;
          vb = cross_group_sum(vb, g.NG);
          vc = cross_group_sum(vc, g.NG);
          if (lane < g.NG) {
            partB[(tt * g.nwarp + warp) * g.N + lane * 4 + i] = vb;
            partC[(tt * g.nwarp + warp) * g.N + lane * 4 + i] = vc;
          }
        }
        {
          // both clock partials in one butterfly: lanes 0..15 end with the ddelta sum, lanes 16..31 with the dlam sum
          const bool up = (lane & 16) != 0;
          float k = up ? sL : sD;
          k += __shfl_xor_sync(0xffffffffu, up ? sD : sL, 16);
#pragma unroll
          for (int o = 8; o > 0; o >>= 1) k += __shfl_xor_sync(0xffffffffu, k, o);
          if ((lane & 15) == 0) partS[(tt * g.nwarp + warp) * 2 + (up ? 1 : 0)] = k;
        }
      }
      }   // half
      __syncthreads();
      // ---- finish the sub-chunk: sum the per-warp partials in warp order
      // A warp holds 32 / NG channel groups; when NG == 32 lanes map 1:1 to row groups.  Rows n = ng * 4 + i.
      for (int idx = tid; idx < 8 * g.N; idx += blockDim.x) {
        const int tt = idx / g.N, n = idx % g.N;
        float sb = 0.f, sc = 0.f;
        for (int w = 0; w < g.nwarp; ++w) { sb += partB[(tt * g.nwarp + w) * g.N + n]; sc += partC[(tt * g.nwarp + w) * g.N + n]; }
        partB[(tt * g.nwarp) * g.N + n] = sb;      // slot of warp 0 now holds the total
        partC[(tt * g.nwarp) * g.N + n] = sc;
      }
      __syncthreads();
      if (tid < g.K) {
        // back through the rotation, newest token first (suffix sum of the phase gradient)
        const int k = tid;
        float S = Ssuf[k];
        for (int tt = HM_TT - 1; tt >= 0; --tt) {
          const int tok = t0 + tt;
          if (tok >= a.L) { phs[tt * g.K + k] = 0.f; continue; }
          float* gb = partB + (tt * g.nwarp) * g.N + 2 * k;
          float* gc = partC + (tt * g.nwarp) * g.N + 2 * k;
          float ph = 0.f;
          if (a.feat != nullptr && a.rot[k]) {
            const int r = tt + 1;
            const float B0 = tl.Bt[r * g.N + 2 * k], B1 = tl.Bt[r * g.N + 2 * k + 1];
            const float C0 = tl.Ct[r * g.N + 2 * k], C1 = tl.Ct[r * g.N + 2 * k + 1];
            const float dthB = gb[1] * B0 - gb[0] * B1, dthC = gc[1] * C0 - gc[0] * C1;
            const float cb = tl.cB[r * g.K + k], sb = tl.sB[r * g.K + k], cc = tl.cC[r * g.K + k], sc = tl.sC[r * g.K + k];
            const float g0 = gb[0] * cb + gb[1] * sb, g1 = -gb[0] * sb + gb[1] * cb;
            const float e0 = gc[0] * cc + gc[1] * sc, e1 = -gc[0] * sc + gc[1] * cc;
            gb[0] = g0; gb[1] = g1; gc[0] = e0; gc[1] = e1;
            acc_th += dthC;
            S += dthB + dthC;
            const float ft = raw[(seq + 1) & 1].feat[tt * g.K + k];      // this tile's staged copy (seq already advanced)
            ph = ft * S;
            if (a.dfeat_part) a.dfeat_part[(((int64_t)h * a.B + b) * a.L + tok) * g.K + k] = tl.dts[r] * S;
          } else if (a.dfeat_part) {
            a.dfeat_part[(((int64_t)h * a.B + b) * a.L + tok) * g.K + k] = 0.f;
          }
          phs[tt * g.K + k] = ph;
        }
        Ssuf[k] = S;
      }
      __syncthreads();
      if (tid < g.N) {
        for (int tt = 0; tt < HM_TT; ++tt) {
          const int tok = t0 + tt;
          if (tok >= a.L) break;
          const float vb = partB[(tt * g.nwarp) * g.N + tid], vc = partC[(tt * g.nwarp) * g.N + tid];
          a.dBh_part[(((int64_t)h * a.B + b) * a.L + tok) * g.N + tid] = vb;
          a.dCh_part[(((int64_t)h * a.B + b) * a.L + tok) * g.N + tid] = vc;
          acc_bb += vb;
          acc_bc += vc;
        }
      }
      if (tid < HM_TT && t0 + tid < a.L) {
        const int tt = tid, tok = t0 + tt;
        float sD = 0.f, sL = 0.f;
        for (int w = 0; w < g.nwarp; ++w) { sD += partS[(tt * g.nwarp + w) * 2]; sL += partS[(tt * g.nwarp + w) * 2 + 1]; }
        for (int k = 0; k < g.K; ++k) sD += phs[tt * g.K + k];
        a.ddelta[((int64_t)b * a.L + tok) * a.H + h] = sD;
        if (a.dlam) a.dlam[((int64_t)b * a.L + tok) * a.H + h] = sL;
      }
      for (int idx = tid; idx < HM_TT * g.P; idx += blockDim.x) {
        const int tt = idx / g.P, pp = idx % g.P;
        if (t0 + tt < a.L) stf(dx + ((int64_t)b * a.L + t0 + tt) * a.H * g.P + h * g.P + pp, dxs[idx]);
      }
      if (tid < g.P)
        for (int tt = 0; tt < HM_TT; ++tt) acc_D = fmaf(tl.dys[tt * g.P + tid], tl.xs[(tt + 1) * g.P + tid], acc_D);
      __syncthreads();
    }
  }
  // ---- what is left after token 0
  if (th.active) {
    if (a.dh_init) store16(G, a.dh_init + bh * PN, th, g.N);
    if (a.dwrite_prev) {
      float wv[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) wv[e] = lagn * G[e];
      store16(wv, a.dwrite_prev + bh * PN, th, g.N);
    }
#pragma unroll
    for (int e = 0; e < 16; ++e) dA[e] *= HM_LN2;       // the sums were taken with rate2 = rate log2(e)
    store16(dA, a.dA_log_part + bh * PN, th, g.N);
  }
  if (tid < g.N) {
    if (a.dbeta_b_part) a.dbeta_b_part[bh * g.N + tid] = acc_bb;
    if (a.dbeta_c_part) a.dbeta_c_part[bh * g.N + tid] = acc_bc;
  }
  if (tid < g.K) {
    if (a.dtheta_h_part) a.dtheta_h_part[bh * g.K + tid] = acc_th;
    if (a.dtheta_init) a.dtheta_init[bh * g.K + tid] = Ssuf[tid];
  }
  if (a.dD_part != nullptr) {
    const float tot = block_sum(tid < g.P ? acc_D : 0.f, red);
    if (tid == 0) a.dD_part[bh] = tot;
  }
}

// ---------------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------------
static int hm_check(const HmArgs* a, int dtype, const char* who, bool bwd) {
  ORBIT_REQUIRE(a != nullptr, ERR_BAD_ARG, "%s: null argument block", who);
  ORBIT_REQUIRE(dtype == F32 || dtype == BF16, ERR_BAD_ARG, "%s: unknown dtype code %d", who, dtype);
  ORBIT_REQUIRE(a->B > 0 && a->L > 0 && a->H > 0 && a->P > 0 && a->N > 0, ERR_BAD_ARG, "%s: bad geometry B=%d L=%d H=%d P=%d N=%d",
                who, a->B, a->L, a->H, a->P, a->N);
  const int NG = a->N / 4;
  ORBIT_REQUIRE(a->P % 4 == 0 && a->N % 4 == 0 && NG <= 32 && (NG & (NG - 1)) == 0 && (a->P / 4) * NG <= 256, ERR_UNSUPPORTED,
                "%s: serves P and N multiples of 4 with N/4 a power of two <= 32 and (P/4)(N/4) <= 256, got P=%d N=%d", who, a->P, a->N);
  ORBIT_REQUIRE(a->x && a->delta && a->A_log && a->Bh && a->Ch, ERR_BAD_ARG, "%s: null x/delta/A_log/Bh/Ch", who);
  ORBIT_REQUIRE(a->feat == nullptr || a->rot != nullptr, ERR_BAD_ARG, "%s: feat needs the rot mask", who);
  ORBIT_REQUIRE(a->Tc > 0 && a->Tc % HM_TT == 0 && a->nck == (a->L + a->Tc - 1) / a->Tc, ERR_BAD_ARG,
                "%s: Tc=%d must be a multiple of %d and nck=%d must equal ceil(L/Tc)", who, a->Tc, HM_TT, a->nck);
  ORBIT_REQUIRE(aligned16(a->A_log) && (!a->h_init || aligned16(a->h_init)) && (!a->write_prev || aligned16(a->write_prev)) &&
                    (!a->hck || aligned16(a->hck)),
                ERR_UNSUPPORTED, "%s: A_log, h_init, write_prev, hck must be 16-byte aligned", who);
  if (!bwd) {
    ORBIT_REQUIRE(a->y && a->h_final && aligned16(a->h_final) && (!a->write_last || aligned16(a->write_last)), ERR_BAD_ARG,
                  "%s: null y/h_final or misaligned state output", who);
  } else {
    ORBIT_REQUIRE(a->Tc == HM_TC, ERR_UNSUPPORTED, "%s: the backward is written for Tc=%d", who, HM_TC);
    ORBIT_REQUIRE(a->dy && a->dx && a->ddelta && a->dA_log_part && a->dBh_part && a->dCh_part && a->hck, ERR_BAD_ARG,
                  "%s: null dy/dx/ddelta/dA_log_part/dBh_part/dCh_part/hck", who);
    ORBIT_REQUIRE(a->feat == nullptr || a->thck != nullptr, ERR_BAD_ARG, "%s: rotation needs thck", who);
    ORBIT_REQUIRE(aligned16(a->dA_log_part) && (!a->dh_final || aligned16(a->dh_final)) && (!a->dh_init || aligned16(a->dh_init)) &&
                      (!a->dwrite_prev || aligned16(a->dwrite_prev)),
                  ERR_UNSUPPORTED, "%s: state gradients must be 16-byte aligned", who);
  }
  return OK;
}

static size_t hm_smem_fwd(const HmGeo& g) { return sizeof(float) * (hm_tile_floats(g, false) + 8 * g.P + 2 * hm_raw_floats(g)); }
static size_t hm_smem_bwd(const HmGeo& g) {
  return sizeof(float) * (hm_tile_floats(g, true) + (size_t)HM_SUB * g.P * g.N + r4(HM_SUB * g.K) + 2 * 8 * g.nwarp * g.N +
                          8 * g.nwarp * 2 + 8 * g.P + 8 * g.K + r4(g.K) + 32 + 2 * hm_raw_floats(g));
}

}  // namespace orbit

using namespace orbit;

extern "C" int orbit_hm_scan_fwd(const orbit_hm_args* a, int dtype, void* stream) {
  int rc = hm_check(a, dtype, "orbit_hm_scan_fwd", false);
  if (rc != OK) return rc;
  const HmGeo g = hm_geo(a->P, a->N);
  const size_t smem = hm_smem_fwd(g);
  ORBIT_REQUIRE(smem <= 200 * 1024, ERR_UNSUPPORTED, "orbit_hm_scan_fwd: tile needs %zu bytes of shared memory", smem);
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid(a->H, a->B);
  auto go = [&](auto kernel) -> int {
    ORBIT_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kernel<<<grid, g.nthr, smem, st>>>(*a);
    return OK;
  };
  const bool trap = a->lam != nullptr;
  rc = dtype == BF16 ? (trap ? go(hm_fwd_kernel<__nv_bfloat16, true>) : go(hm_fwd_kernel<__nv_bfloat16, false>))
                     : (trap ? go(hm_fwd_kernel<float, true>) : go(hm_fwd_kernel<float, false>));
  if (rc != OK) return rc;
  ORBIT_CHECK_LAUNCH("hm_fwd_kernel");
  return OK;
}

extern "C" int orbit_hm_scan_bwd(const orbit_hm_args* a, int dtype, void* stream) {
  int rc = hm_check(a, dtype, "orbit_hm_scan_bwd", true);
  if (rc != OK) return rc;
  const HmGeo g = hm_geo(a->P, a->N);
  const size_t smem = hm_smem_bwd(g);
  ORBIT_REQUIRE(smem <= 220 * 1024, ERR_UNSUPPORTED, "orbit_hm_scan_bwd: P=%d, N=%d need %zu bytes of shared memory (limit 220 KiB)",
                a->P, a->N, smem);
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid(a->H, a->B);
  auto go = [&](auto kernel) -> int {
    ORBIT_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kernel<<<grid, g.nthr, smem, st>>>(*a);
    return OK;
  };
  const bool trap = a->lam != nullptr;
  rc = dtype == BF16 ? (trap ? go(hm_bwd_kernel<__nv_bfloat16, true>) : go(hm_bwd_kernel<__nv_bfloat16, false>))
                     : (trap ? go(hm_bwd_kernel<float, true>) : go(hm_bwd_kernel<float, false>));
  if (rc != OK) return rc;
  ORBIT_CHECK_LAUNCH("hm_bwd_kernel");
  return OK;
}

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
// A thread owns 4 channels x NJ rows of the state (NJ = 4, or 2 for twice the threads at half the registers each).
__host__ __device__ constexpr HmGeo hm_geo(int P, int N, int NJ = 4) {
  HmGeo g{};
  g.P = P; g.N = N; g.K = N / 2; g.NG = N / NJ;
  g.active = (P / 4) * g.NG;
  g.nthr = (g.active + 31) / 32 * 32;
  g.nwarp = g.nthr / 32;
  return g;
}

// Shared-memory tile of 8 tokens (+ the token before them in row 0).
struct HmTile {
  float *xs, *dts, *lams, *Bt, *Ct, *cB, *sB, *cC, *sC, *dys, *thc, *thn;
  float *rotm, *thh, *bb, *bc;     // per-head constants of the builder: rotating-pair mask, phase offset of the C map, map biases
  float *featc;                    // backward: the tile's angle features (its staged copy is gone by the time they are used)
};
__host__ __device__ inline size_t r4(size_t n) { return (n + 3) & ~(size_t)3; }
// Every array starts on a 16-byte boundary (xs, Bt, Ct, dys rows are read as float4).
// The forward kernel has one tile; the backward with compile-time geometry keeps the tiles of a chunk's four sub-chunks
// (built once, in the chunk's replay, and used again by the reverse walk); with run-time geometry, where four tiles may
// not fit the shared memory, it has one tile and builds a sub-chunk's tile again for the reverse walk.  Shared between
// the tiles: the running phase and the per-head constants.
__host__ __device__ inline size_t hm_slot_floats(const HmGeo& g, bool bwd) {
  size_t n = 9 * g.P + 9 * g.N + 9 * g.N + 12 + 12;
  if (bwd) n += 8 * g.P + 4 * r4(9 * g.K) + r4(8 * g.K);
  return n;
}
__host__ __device__ inline size_t hm_tile_floats(const HmGeo& g, bool bwd, int slots = 1) {
  return 4 * r4(g.K) + 2 * g.N + slots * hm_slot_floats(g, bwd);
}
// point the per-tile arrays of `t` at slot `j` of the tile area `base`
__device__ __forceinline__ void hm_tile_slot(HmTile& t, float* base, int j, const HmGeo& g, bool bwd) {
  float* p = base + (size_t)j * hm_slot_floats(g, bwd);
  t.xs = p; p += 9 * g.P;
  t.Bt = p; p += 9 * g.N;
  t.Ct = p; p += 9 * g.N;
  t.dts = p; p += 12;
  t.lams = p; p += 12;
  t.cB = t.sB = t.cC = t.sC = t.dys = t.featc = nullptr;
  if (bwd) {
    t.dys = p; p += 8 * g.P;
    t.cB = p; p += r4(9 * g.K);
    t.sB = p; p += r4(9 * g.K);
    t.cC = p; p += r4(9 * g.K);
    t.sC = p; p += r4(9 * g.K);
    t.featc = p;
  }
}
// carve the shared arrays and the tile area (slot 0 selected); returns the first float after the area
__device__ inline float* hm_tile_carve(HmTile& t, float* p, const HmGeo& g, bool bwd, float** area = nullptr, int slots = 1) {
  t.thc = p; p += r4(g.K);
  t.thn = p; p += r4(g.K);
  t.rotm = p; p += r4(g.K);
  t.thh = p; p += r4(g.K);
  t.bb = p; p += g.N;
  t.bc = p; p += g.N;
  if (area != nullptr) *area = p;
  hm_tile_slot(t, p, 0, g, bwd);
  return p + slots * hm_slot_floats(g, bwd);
}
// The per-head constants, written once per CTA (the opening barrier of the first tile build publishes them).
__device__ __forceinline__ void hm_tile_consts(const HmArgs& a, const HmGeo& g, const HmTile& tl, int h) {
  for (int k = threadIdx.x; k < g.K; k += blockDim.x) {
    tl.rotm[k] = (a.feat != nullptr && a.rot[k]) ? 1.f : 0.f;
    tl.thh[k] = a.theta_h ? a.theta_h[h * g.K + k] : 0.f;
  }
  for (int n = threadIdx.x; n < g.N; n += blockDim.x) {
    tl.bb[n] = a.beta_b ? a.beta_b[h * g.N + n] : 0.f;
    tl.bc[n] = a.beta_c ? a.beta_c[h * g.N + n] : 0.f;
  }
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
__device__ __forceinline__ void cp_async16s(uint32_t smem_dst, const void* gsrc, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gsrc), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Staging plan of a tile in 16-byte units.  Which unit copies what is the same for every tile of a CTA, so the split of a
// unit index into (array, row, column) is done once and kept in shared memory: unit u = {destination byte offset inside
// the raw buffer | array << 24 | (row's token offset + 1) << 28, source byte offset inside the token's row}.
// Arrays: 0 drive, 1 dy, 2 B map, 3 C map, 4 angle feature.  Used when every row is a whole number of 16-byte units and
// every base pointer is 16-byte aligned; otherwise the tile is staged word by word.
struct HmPlan {
  const uint2* unit;
  int n;
  bool vec;
};
__host__ __device__ inline size_t hm_plan_floats(const HmGeo& g) {      // sized for 4-byte elements (the upper bound)
  return r4(2 * ((size_t)17 * (g.P / 4) + 18 * (g.N / 4) + 8 * ((g.K + 3) / 4)));
}
template <typename T, bool BWD>
__device__ __forceinline__ HmPlan hm_plan_build(const HmArgs& a, const HmGeo& g, uint2* tab, const HmRaw& rw) {
  HmPlan pl;
  pl.unit = tab;
  constexpr int esz = (int)sizeof(T);
  const int nux = g.P * esz / 16, nun = g.N / 4, nuk = g.K / 4;
  uintptr_t al = (uintptr_t)a.x | (uintptr_t)a.Bh | (uintptr_t)a.Ch;
  if (BWD) al |= (uintptr_t)a.dy;
  if (a.feat != nullptr) al |= (uintptr_t)a.feat;
  pl.vec = (g.P * esz) % 16 == 0 && g.N % 8 == 0 && (al & 15) == 0;
  const int n0 = 9 * nux, n1 = n0 + (BWD ? 8 * nux : 0), n2 = n1 + 9 * nun, n3 = n2 + 9 * nun, n4 = n3 + (a.feat != nullptr ? 8 * nuk : 0);
  pl.n = pl.vec ? n4 : 0;
  for (int u = threadIdx.x; u < pl.n; u += blockDim.x) {
    int kind, r, c, dr;
    uint32_t dst;
    if (u < n0) {
      kind = 0; r = u / nux; c = u % nux; dr = r - 1;
      dst = (uint32_t)(r * g.P * esz + c * 16);
    } else if (u < n1) {
      const int v = u - n0;
      kind = 1; r = v / nux; c = v % nux; dr = r;
      dst = (uint32_t)(rw.dy - rw.x) + (uint32_t)(r * g.P * esz + c * 16);
    } else if (u < n2) {
      const int v = u - n1;
      kind = 2; r = v / nun; c = v % nun; dr = r - 1;
      dst = (uint32_t)(reinterpret_cast<const unsigned char*>(rw.B) - rw.x) + (uint32_t)((r * g.N + c * 4) * 4);
    } else if (u < n3) {
      const int v = u - n2;
      kind = 3; r = v / nun; c = v % nun; dr = r - 1;
      dst = (uint32_t)(reinterpret_cast<const unsigned char*>(rw.C) - rw.x) + (uint32_t)((r * g.N + c * 4) * 4);
    } else {
      const int v = u - n3;
      kind = 4; r = v / nuk; c = v % nuk; dr = r;
      dst = (uint32_t)(reinterpret_cast<const unsigned char*>(rw.feat) - rw.x) + (uint32_t)((r * g.K + c * 4) * 4);
    }
    tab[u] = make_uint2(dst | ((uint32_t)kind << 24) | ((uint32_t)(dr + 1) << 28), (uint32_t)(c * 16));
  }
  return pl;
}

// Issue the copies of tokens [t0 - 1, t0 + 8) (t0 < 0: nothing).  Tokens outside [0, L) are zero-filled.
template <typename T, bool BWD>
__device__ __forceinline__ void hm_prefetch(const HmArgs& a, const HmGeo& g, const HmPlan& pl, const HmRaw& rw, int b, int h, int t0) {
  if (t0 >= 0) {
    const int tid = threadIdx.x, nt = blockDim.x;
    if (pl.vec) {
      const uint32_t base = (uint32_t)__cvta_generic_to_shared(rw.x);
      const int64_t bl = (int64_t)b * a.L;
      const int64_t sx = (int64_t)a.H * g.P * (int)sizeof(T), sn = (int64_t)g.N * 4, sk = (int64_t)g.K * 4;   // bytes per token
      const char* px = reinterpret_cast<const char*>(a.x) + (int64_t)h * g.P * (int)sizeof(T);
      const char* pdy = BWD ? reinterpret_cast<const char*>(a.dy) + (int64_t)h * g.P * (int)sizeof(T) : px;
      for (int u = tid; u < pl.n; u += nt) {
        const uint2 d = pl.unit[u];
        const int kind = (int)(d.x >> 24) & 7, tok = t0 + (int)(d.x >> 28) - 1;
        const bool ok = tok >= 0 && tok < a.L;
        const int64_t row = bl + (ok ? tok : 0);
        const char* src = kind == 0   ? px + row * sx
                          : kind == 1 ? pdy + row * sx
                          : kind == 2 ? reinterpret_cast<const char*>(a.Bh) + row * sn
                          : kind == 3 ? reinterpret_cast<const char*>(a.Ch) + row * sn
                                      : reinterpret_cast<const char*>(a.feat) + row * sk;
        cp_async16s(base + (d.x & 0xffffffu), src + d.y, ok);
      }
    } else {
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

// sin and cos of a running phase.  Phases of this size are first brought to [-pi, pi] (two-constant reduction: 6.28125 is
// exact in 8 bits, so k * 6.28125 is exact for every k that can occur), where the MUFU sine and cosine are good to 4e-7
// absolute; anything larger takes the library's full-range path.
__device__ __forceinline__ void phase_sincos(float x, float* s, float* c) {
  if (fabsf(x) > 8192.f) {
    sincosf(x, s, c);
    return;
  }
  const float k = rintf(x * 0.15915494309189535f);
  float r = fmaf(k, -6.28125f, x);
  r = fmaf(k, -1.9353071795864769e-3f, r);
  *s = __sinf(r);
  *c = __cosf(r);
}

// Build the tile of tokens [t0 - 1, t0 + 8) from its staged raw copy.  tile.thc holds the phase entering token t0 and
// leaves holding the phase after token t0 + 7.  Two barriers: one before the raw copy is read, one after the tile is
// written.  Every (row, pair) item forms its own phase, the running sum from the entering phase in token order (row r
// takes the first r terms), so no item waits for another; the item of the last row leaves the next entering phase.
// eight consecutive elements of the IO dtype -> fp32 (both addresses 16-byte aligned)
__device__ __forceinline__ void cvt8(float* dst, const float* src) {
  *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(src);
  *reinterpret_cast<float4*>(dst + 4) = *reinterpret_cast<const float4*>(src + 4);
}
__device__ __forceinline__ void cvt8(float* dst, const __nv_bfloat16* src) {
  const uint4 v = *reinterpret_cast<const uint4*>(src);
  float f[8];
  unpack_bf16(v.x, f[0], f[1]); unpack_bf16(v.y, f[2], f[3]); unpack_bf16(v.z, f[4], f[5]); unpack_bf16(v.w, f[6], f[7]);
  *reinterpret_cast<float4*>(dst) = make_float4(f[0], f[1], f[2], f[3]);
  *reinterpret_cast<float4*>(dst + 4) = make_float4(f[4], f[5], f[6], f[7]);
}

template <typename T, bool BWD>
__device__ __forceinline__ void hm_build_tile(const HmArgs& a, const HmGeo& g, HmTile& tl, const HmRaw& rw, int b, int h, int t0) {
  const int tid = threadIdx.x, nt = blockDim.x;
  cp_async_wait_all();
  __syncthreads();
  const T* rx = reinterpret_cast<const T*>(rw.x);
  const T* rdy = reinterpret_cast<const T*>(rw.dy);
  if (g.P % 8 == 0) {
    const int nx = 9 * g.P / 8, ny = BWD ? 8 * g.P / 8 : 0;
    for (int idx = tid; idx < nx + ny; idx += nt) {
      if (idx < nx) cvt8(tl.xs + idx * 8, rx + idx * 8);
      else cvt8(tl.dys + (idx - nx) * 8, rdy + (idx - nx) * 8);
    }
  } else {
    for (int idx = tid; idx < 9 * g.P; idx += nt) tl.xs[idx] = ldf(rx + idx);
    if (BWD)
      for (int idx = tid; idx < 8 * g.P; idx += nt) tl.dys[idx] = ldf(rdy + idx);
  }
  if (tid < 9) {
    tl.dts[tid] = rw.dt[tid];
    tl.lams[tid] = a.lam ? rw.lam[tid] : 1.f;
  }
  const bool rotating = a.feat != nullptr;
  if (BWD && rotating)
    for (int idx = tid; idx < 8 * g.K; idx += nt) tl.featc[idx] = rw.feat[idx];
  const int lgK = 31 - __clz(g.K);                      // K = N / 2 is a power of two
  // Rows 1..8 (the tile's tokens): both maps.  Row r sees the phase after token t0 + r - 1 (clocks and features are
  // zero-filled past the end of the sequence).
  for (int idx = tid; idx < 8 * g.K; idx += nt) {
    const int r = 1 + (idx >> lgK), k = idx & (g.K - 1), tok = t0 - 1 + r;
    float b0 = 0.f, b1 = 0.f, c0 = 0.f, c1 = 0.f;
    if (tok < a.L) {
      const float2 bv = *reinterpret_cast<const float2*>(rw.B + r * g.N + 2 * k), cv = *reinterpret_cast<const float2*>(rw.C + r * g.N + 2 * k);
      const float2 bbv = *reinterpret_cast<const float2*>(tl.bb + 2 * k), bcv = *reinterpret_cast<const float2*>(tl.bc + 2 * k);
      b0 = bv.x + bbv.x; b1 = bv.y + bbv.y; c0 = cv.x + bcv.x; c1 = cv.y + bcv.y;
    }
    float cb = 1.f, sb = 0.f, cc = 1.f, sc = 0.f;
    if (rotating) {
      float th = tl.thc[k];
#pragma unroll
      for (int j = 1; j <= 8; ++j)
        if (j <= r) th = fmaf(rw.dt[j], rw.feat[(j - 1) * g.K + k], th);
      if (r == 8) tl.thn[k] = th;
      if (tl.rotm[k] != 0.f) {
        phase_sincos(th, &sb, &cb);
        phase_sincos(th + tl.thh[k], &sc, &cc);
      }
    }
    *reinterpret_cast<float2*>(tl.Bt + r * g.N + 2 * k) = make_float2(b0 * cb - b1 * sb, b0 * sb + b1 * cb);
    *reinterpret_cast<float2*>(tl.Ct + r * g.N + 2 * k) = make_float2(c0 * cc - c1 * sc, c0 * sc + c1 * cc);
    if (BWD) { const int o = r * g.K + k; tl.cB[o] = cb; tl.sB[o] = sb; tl.cC[o] = cc; tl.sC[o] = sc; }
  }
  // Row 0 (token t0 - 1, at the entering phase): only its B map is ever read (the previous token's write of the trapezoid
  // rule).  Dealt from the last thread down, so that it does not land on the warp that gets the first rows again.
  for (int k = nt - 1 - tid; k < g.K; k += nt) {
    float b0 = 0.f, b1 = 0.f;
    if (t0 >= 1) {
      const float2 bv = *reinterpret_cast<const float2*>(rw.B + 2 * k), bbv = *reinterpret_cast<const float2*>(tl.bb + 2 * k);
      b0 = bv.x + bbv.x; b1 = bv.y + bbv.y;
    }
    float cb = 1.f, sb = 0.f;
    if (rotating && tl.rotm[k] != 0.f) phase_sincos(tl.thc[k], &sb, &cb);
    *reinterpret_cast<float2*>(tl.Bt + 2 * k) = make_float2(b0 * cb - b1 * sb, b0 * sb + b1 * cb);
  }
  __syncthreads();
  if (rotating) {
    float* t = tl.thc;
    tl.thc = tl.thn;
    tl.thn = t;
  }
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
template <int NJ>
__device__ __forceinline__ void load_rows(float (&v)[NJ], const float* p) {
  if constexpr (NJ == 4) {
    const float4 r = *reinterpret_cast<const float4*>(p);
    v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
  } else {
    const float2 r = *reinterpret_cast<const float2*>(p);
    v[0] = r.x; v[1] = r.y;
  }
}
template <bool TRAP, int NJ>
__device__ __forceinline__ void hm_step(float (&hs)[4 * NJ], float (&prv)[4 * NJ], const float (&rate2)[4 * NJ], const float4 x4,
                                        const float (&bv)[NJ], float d, float lm) {
  // two rows at a time (packed fp32): the per-element work of these kernels is bound by instruction issue
  const float xv[4] = {x4.x, x4.y, x4.z, x4.w};
  const float dl = d * lm, dg = d * (1.f - lm);
  const float2 d2 = make_float2(d, d), dl2 = make_float2(dl, dl), dg2 = make_float2(dg, dg);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 x2 = make_float2(xv[i], xv[i]);
#pragma unroll
    for (int j = 0; j < NJ; j += 2) {
      const int e = i * NJ + j;
      const float2 rd = mul2(make_float2(rate2[e], rate2[e + 1]), d2);
      const float2 av = make_float2(fast_ex2(rd.x), fast_ex2(rd.y));
      const float2 raw = mul2(x2, make_float2(bv[j], bv[j + 1]));
      float2 h2 = make_float2(hs[e], hs[e + 1]);
      if (TRAP) h2 = fma2(av, fma2(dg2, make_float2(prv[e], prv[e + 1]), h2), mul2(dl2, raw));
      else h2 = fma2(av, h2, mul2(d2, raw));
      hs[e] = h2.x; hs[e + 1] = h2.y;
      prv[e] = raw.x; prv[e + 1] = raw.y;
    }
  }
}

// the thread's 4 x NJ tile of a [P, N] array
template <int NJ>
__device__ __forceinline__ void load_tile(float (&v)[4 * NJ], const float* base, const HmThread& th, int N) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float r[NJ];
    load_rows<NJ>(r, base + (int64_t)(th.pg * 4 + i) * N + th.ng * NJ);
#pragma unroll
    for (int j = 0; j < NJ; ++j) v[i * NJ + j] = r[j];
  }
}
template <int NJ>
__device__ __forceinline__ void store_tile(const float (&v)[4 * NJ], float* base, const HmThread& th, int N) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float* q = base + (int64_t)(th.pg * 4 + i) * N + th.ng * NJ;
    if constexpr (NJ == 4) *reinterpret_cast<float4*>(q) = make_float4(v[i * 4], v[i * 4 + 1], v[i * 4 + 2], v[i * 4 + 3]);
    else *reinterpret_cast<float2*>(q) = make_float2(v[i * 2], v[i * 2 + 1]);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------------------------
// CP, CN > 0: the geometry P, N as compile-time constants (every shared-memory offset and index split folds away, which
// is worth tens of registers); 0: read from the arguments.
template <typename T, bool TRAP, int CP, int CN>
__global__ void __launch_bounds__(256) hm_fwd_kernel(const HmArgs a) {
  extern __shared__ __align__(16) float smf[];
  const HmGeo g = CP > 0 ? hm_geo(CP, CN) : hm_geo(a.P, a.N);
  HmTile tl;
  float* ys = hm_tile_carve(tl, smf, g, false);      // [8][P]
  HmRaw raw[2];
  float* rp = hm_raw_carve(raw[0], ys + 8 * g.P, g);
  rp = hm_raw_carve(raw[1], rp, g);
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
  const HmPlan plan = hm_plan_build<T, false>(a, g, reinterpret_cast<uint2*>(rp), raw[0]);
  hm_tile_consts(a, g, tl, h);
  __syncthreads();
  hm_prefetch<T, false>(a, g, plan, raw[0], b, h, 0);
  const HmThread th = hm_thread(g);
  constexpr bool trap = TRAP;
  const int64_t bh = (int64_t)b * a.H + h;
  float hs[16], prv[16], rate[16];
  load_tile<4>(rate, a.A_log + (int64_t)h * g.P * g.N, th, g.N);
#pragma unroll
  for (int e = 0; e < 16; ++e) { rate[e] = -__expf(rate[e]) * HM_LOG2E; hs[e] = 0.f; prv[e] = 0.f; }
  if (a.h_init) load_tile<4>(hs, a.h_init + bh * g.P * g.N, th, g.N);
  if (a.write_prev && trap) load_tile<4>(prv, a.write_prev + bh * g.P * g.N, th, g.N);
  if (tid < g.K) tl.thc[tid] = a.theta_init ? a.theta_init[bh * g.K + tid] : 0.f;
  const float Dh = a.D ? a.D[h] : 0.f;
  __syncthreads();
  T* y = (T*)a.y;
  for (int t0 = 0; t0 < a.L; t0 += HM_TT) {
    if (a.hck != nullptr && t0 % a.Tc == 0) {
      const int c = t0 / a.Tc;
      if (th.active) store_tile<4>(hs, a.hck + (bh * a.nck + c) * g.P * g.N, th, g.N);
      if (a.thck != nullptr && tid < g.K) a.thck[(bh * a.nck + c) * g.K + tid] = tl.thc[tid];
    }
    const int it = t0 / HM_TT;
    hm_build_tile<T, false>(a, g, tl, raw[it & 1], b, h, t0);
    hm_prefetch<T, false>(a, g, plan, raw[(it + 1) & 1], b, h, t0 + HM_TT < a.L ? t0 + HM_TT : -1);
    const int nv = min(HM_TT, a.L - t0);
#pragma unroll
    for (int tt = 0; tt < HM_TT; ++tt) {
      if (tt < nv) {
        const float4 x4 = *reinterpret_cast<const float4*>(tl.xs + (tt + 1) * g.P + th.pg * 4);
        float bv[4], cv[4];
        load_rows<4>(bv, tl.Bt + (tt + 1) * g.N + th.ng * 4);
        load_rows<4>(cv, tl.Ct + (tt + 1) * g.N + th.ng * 4);
        hm_step<TRAP, 4>(hs, prv, rate, x4, bv, tl.dts[tt + 1], tl.lams[tt + 1]);
        const float xv[4] = {x4.x, x4.y, x4.z, x4.w};
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
    store_tile<4>(hs, a.h_final + bh * g.P * g.N, th, g.N);
    if (a.write_last) store_tile<4>(prv, a.write_last + bh * g.P * g.N, th, g.N);
  }
  if (a.theta_final != nullptr && tid < g.K) a.theta_final[bh * g.K + tid] = tl.thc[tid];
}

// ---------------------------------------------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------------------------------------------
// NJ = rows of the state per thread (4 x NJ tile).  CP, CN as in the forward kernel.
template <typename T, bool TRAP, int NJ, int CP, int CN>
__global__ void __launch_bounds__(NJ == 2 ? 512 : 256, 1) hm_bwd_kernel(const HmArgs a) {
  constexpr int E = 4 * NJ;
  extern __shared__ __align__(16) float smf[];
  const HmGeo g = CP > 0 ? hm_geo(CP, CN, NJ) : hm_geo(a.P, a.N, NJ);
  constexpr bool CACHE = CP > 0;          // keep the four tiles of a chunk (see hm_slot_floats)
  HmTile tl;
  float* tiles;
  float* p = hm_tile_carve(tl, smf, g, true, &tiles, CACHE ? HM_SUB : 1);
  float* hsub = p;  p += (size_t)HM_SUB * g.P * g.N;     // state entering each sub-chunk of the current chunk
  float* thsub = p; p += r4(HM_SUB * g.K);               // phase entering each sub-chunk (used when the tiles are rebuilt)
  float* partB = p; p += 8 * g.nwarp * g.N;              // [tt][warp][n]
  float* partC = p; p += 8 * g.nwarp * g.N;
  float* partS = p; p += 8 * g.nwarp * 2;                // [tt][warp][ddelta, dlam]
  float* dxs = p;   p += 8 * g.P;
  float* phs = p;   p += 8 * g.K;                        // [tt][k] phase gradient of the token, then feat * suffix (phase part of ddelta)
  float* dcs = p;   p += 8 * g.K;                        // [tt][k] the C map's share of the phase gradient (-> dtheta_h)
  float* Ssuf = p;  p += r4(g.K);                          // suffix sum of dTheta carried backwards in time
  float* red = p;   p += 32;
  HmRaw raw[2];
  p = hm_raw_carve(raw[0], p, g);
  p = hm_raw_carve(raw[1], p, g);
  const HmPlan plan = hm_plan_build<T, true>(a, g, reinterpret_cast<uint2*>(p), raw[0]);
  hm_tile_consts(a, g, tl, blockIdx.x);
  __syncthreads();
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // The tiles are staged in a fixed order, chunks from the last to the first.  With kept tiles: the sub-chunks of a chunk
  // forwards, once.  With rebuilt tiles: the first nsub - 1 sub-chunks forwards (replay), then all nsub backwards.
  // item_t0(c, k) = first token of the k-th tile of chunk c, continuing into chunk c - 1.
  auto n_sub = [&](int c) { return min(HM_SUB, (a.L - c * HM_TC + HM_TT - 1) / HM_TT); };
  auto item_t0 = [&](int c, int k) -> int {
    int ns = n_sub(c);
    if (k >= (CACHE ? ns : 2 * ns - 1)) {
      c -= 1;
      k = 0;
      if (c < 0) return -1;
      ns = HM_SUB;
    }
    if (CACHE) return c * HM_TC + k * HM_TT;
    return c * HM_TC + (k < ns - 1 ? k : (ns - 1) - (k - (ns - 1))) * HM_TT;
  };
  int seq = 0;
  hm_prefetch<T, true>(a, g, plan, raw[0], b, h, item_t0(a.nck - 1, 0));
  const HmThread th = hm_thread(g);
  constexpr bool trap = TRAP;
  const int64_t bh = (int64_t)b * a.H + h;
  const int64_t PN = (int64_t)g.P * g.N;
  float rate[E], G[E], dA[E];
  load_tile<NJ>(rate, a.A_log + (int64_t)h * PN, th, g.N);
#pragma unroll
  for (int e = 0; e < E; ++e) { rate[e] = -__expf(rate[e]) * HM_LOG2E; G[e] = 0.f; dA[e] = 0.f; }
  if (a.dh_final) load_tile<NJ>(G, a.dh_final + bh * PN, th, g.N);
  if (tid < g.K) Ssuf[tid] = a.dtheta_final ? a.dtheta_final[bh * g.K + tid] : 0.f;
  float lagn = 0.f;                       // delta_{t+1} (1 - lam_{t+1}) of the token processed just before (in reverse)
  float acc_bb = 0.f, acc_bc = 0.f;       // the last N threads: dbeta_b[n], dbeta_c[n] of row n = tid - (threads - N)
  float acc_th = 0.f;                     // thread k < K: dtheta_h[k]
  float acc_D = 0.f;                      // thread p < P: partial of dD
  const float Dh = a.D ? a.D[h] : 0.f;
  T* dx = (T*)a.dx;
  __syncthreads();

  for (int c = a.nck - 1; c >= 0; --c) {
    const int tc0 = c * HM_TC;
    int item = 0;
    // ---- replay the chunk once: build the tile of every sub-chunk (kept for the reverse walk) and keep the state that
    // enters each sub-chunk
    {
      float hs[E], prv[E];
      load_tile<NJ>(hs, a.hck + (bh * a.nck + c) * PN, th, g.N);
      if (tid < g.K) tl.thc[tid] = a.thck ? a.thck[(bh * a.nck + c) * g.K + tid] : 0.f;
      __syncthreads();
      const int ns = n_sub(c);
      for (int j = 0; j < ns; ++j) {
        const int t0 = tc0 + j * HM_TT;
        if (th.active) store_tile<NJ>(hs, hsub + (size_t)j * PN, th, g.N);
        if (!CACHE) {
          if (tid < g.K) thsub[j * g.K + tid] = tl.thc[tid];
          if (j == ns - 1) break;          // the last sub-chunk's tile is built by the reverse walk
          hm_build_tile<T, false>(a, g, tl, raw[seq & 1], b, h, t0);
        } else {
          hm_tile_slot(tl, tiles, j, g, true);
          hm_build_tile<T, true>(a, g, tl, raw[seq & 1], b, h, t0);
        }
        ++item;
        ++seq;
        hm_prefetch<T, true>(a, g, plan, raw[seq & 1], b, h, item_t0(c, item));
        if (j == ns - 1) break;            // the last sub-chunk's states are formed by the reverse walk's own replays
        if (j == 0) {
#pragma unroll
          for (int e = 0; e < E; ++e) prv[e] = 0.f;
          if (trap) {
            if (t0 == 0) {
              if (a.write_prev) load_tile<NJ>(prv, a.write_prev + bh * PN, th, g.N);
            } else {
              const float4 x4 = *reinterpret_cast<const float4*>(tl.xs + th.pg * 4);
              const float xv[4] = {x4.x, x4.y, x4.z, x4.w};
              float bv[NJ];
              load_rows<NJ>(bv, tl.Bt + th.ng * NJ);
#pragma unroll
              for (int e = 0; e < E; ++e) prv[e] = xv[e / NJ] * bv[e % NJ];
            }
          }
        }
        const int nv = min(HM_TT, a.L - t0);
        for (int tt = 0; tt < nv; ++tt) {
          const float4 x4 = *reinterpret_cast<const float4*>(tl.xs + (tt + 1) * g.P + th.pg * 4);
          float bv[NJ];
          load_rows<NJ>(bv, tl.Bt + (tt + 1) * g.N + th.ng * NJ);
          hm_step<TRAP, NJ>(hs, prv, rate, x4, bv, tl.dts[tt + 1], tl.lams[tt + 1]);
        }
        if (!CACHE) __syncthreads();       // one tile: every warp is done with it before the next build writes it
      }
      __syncthreads();
    }
    // ---- sub-chunks, last first
    for (int j = HM_SUB - 1; j >= 0; --j) {
      const int t0 = tc0 + j * HM_TT;
      if (t0 >= a.L) continue;
      if (CACHE) {
        hm_tile_slot(tl, tiles, j, g, true);
      } else {
        if (tid < g.K) tl.thc[tid] = thsub[j * g.K + tid];
        __syncthreads();
        hm_build_tile<T, true>(a, g, tl, raw[seq & 1], b, h, t0);
        ++item;
        ++seq;
        hm_prefetch<T, true>(a, g, plan, raw[seq & 1], b, h, item_t0(c, item));
      }
      // The sub-chunk is walked in two halves of 4 tokens (second half first): a half's 4 states are held in registers;
      // the first half is replayed once more from the sub-chunk boundary.  (Keeping all 8 states costs 128 registers
      // and an unrolled body that no longer fits the instruction cache.)
      float hist[4][E];
#pragma unroll 1
      for (int half = 1; half >= 0; --half) {
      float prv0[E];                            // raw write of the token before token 4 * half
      {
        float hs[E], prv[E];
        load_tile<NJ>(hs, hsub + (size_t)j * PN, th, g.N);
#pragma unroll
        for (int e = 0; e < E; ++e) prv[e] = 0.f;
        if (trap) {
          if (t0 == 0) {
            if (a.write_prev) load_tile<NJ>(prv, a.write_prev + bh * PN, th, g.N);
          } else {
            const float4 x4 = *reinterpret_cast<const float4*>(tl.xs + th.pg * 4);
            const float xv[4] = {x4.x, x4.y, x4.z, x4.w};
            float bv[NJ];
            load_rows<NJ>(bv, tl.Bt + th.ng * NJ);
#pragma unroll
            for (int e = 0; e < E; ++e) prv[e] = xv[e / NJ] * bv[e % NJ];
          }
        }
        if (half == 1) {
#pragma unroll
          for (int tt = 0; tt < 4; ++tt) {
            const float4 x4 = *reinterpret_cast<const float4*>(tl.xs + (tt + 1) * g.P + th.pg * 4);
            float bv[NJ];
            load_rows<NJ>(bv, tl.Bt + (tt + 1) * g.N + th.ng * NJ);
            hm_step<TRAP, NJ>(hs, prv, rate, x4, bv, tl.dts[tt + 1], tl.lams[tt + 1]);
          }
        }
#pragma unroll
        for (int e = 0; e < E; ++e) prv0[e] = prv[e];
#pragma unroll
        for (int k = 0; k < 4; ++k) {              // tokens past L: zero clock and drive leave the state unchanged
          const int tt = half * 4 + k;
          const float4 x4 = *reinterpret_cast<const float4*>(tl.xs + (tt + 1) * g.P + th.pg * 4);
          float bv[NJ];
          load_rows<NJ>(bv, tl.Bt + (tt + 1) * g.N + th.ng * NJ);
          hm_step<TRAP, NJ>(hs, prv, rate, x4, bv, tl.dts[tt + 1], tl.lams[tt + 1]);
#pragma unroll
          for (int e = 0; e < E; ++e) hist[k][e] = hs[e];
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
        const float4 dy4 = *reinterpret_cast<const float4*>(tl.dys + tt * g.P + th.pg * 4);
        const float xv[4] = {x4.x, x4.y, x4.z, x4.w}, xpv[4] = {xp4.x, xp4.y, xp4.z, xp4.w};
        const float dyv[4] = {dy4.x, dy4.y, dy4.z, dy4.w};
        float bv[NJ], bpv[NJ], cv[NJ];
        load_rows<NJ>(bv, tl.Bt + (tt + 1) * g.N + th.ng * NJ);
        load_rows<NJ>(bpv, tl.Bt + tt * g.N + th.ng * NJ);
        load_rows<NJ>(cv, tl.Ct + (tt + 1) * g.N + th.ng * NJ);
        float px[4], pB[NJ], pC[NJ];
        float sQ = 0.f, S1 = 0.f, S2 = 0.f;        // sums of dlog rate2, G raw, (a G) raw_prev over this thread's tile
        const float dl = d * lm, dg = d * (1.f - lm);
        const bool last = (tok == a.L - 1) && a.dwrite_last != nullptr;
        if (tok < a.L) {
          // two rows at a time (packed fp32); the pair's lanes are summed where a sum over rows is wanted
          const float2 d2 = make_float2(d, d), dl2 = make_float2(dl, dl), ndl2 = make_float2(-dl, -dl), lag2 = make_float2(lagn, lagn);
          float2 px2[4], pB2[NJ / 2], pC2[NJ / 2];
          float2 sQ2 = make_float2(0.f, 0.f), S12 = sQ2, S22 = sQ2;
#pragma unroll
          for (int jp = 0; jp < NJ / 2; ++jp) { pB2[jp] = make_float2(0.f, 0.f); pC2[jp] = make_float2(0.f, 0.f); }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 dy2 = make_float2(dyv[i], dyv[i]), x2 = make_float2(xv[i], xv[i]), xp2 = make_float2(xpv[i], xpv[i]);
            px2[i] = make_float2(0.f, 0.f);
#pragma unroll
            for (int jp = 0; jp < NJ / 2; ++jp) {
              const int e = i * NJ + 2 * jp;
              const float2 G2 = make_float2(G[e], G[e + 1]), h2 = make_float2(hist[k][e], hist[k][e + 1]);
              const float2 r2 = make_float2(rate[e], rate[e + 1]), b2 = make_float2(bv[2 * jp], bv[2 * jp + 1]);
              const float2 Gt = fma2(make_float2(cv[2 * jp], cv[2 * jp + 1]), dy2, G2);
              pC2[jp] = fma2(dy2, h2, pC2[jp]);
              const float2 raw = mul2(x2, b2);
              const float2 u1 = mul2(Gt, raw);
              const float2 q = mul2(fma2(Gt, h2, mul2(ndl2, u1)), r2);   // dL / d log a_t, times rate2
              const float2 dA2 = fma2(q, d2, make_float2(dA[e], dA[e + 1]));
              dA[e] = dA2.x; dA[e + 1] = dA2.y;
              sQ2 = add2(sQ2, q);
              const float2 rd = mul2(r2, d2);
              const float2 aG = mul2(make_float2(fast_ex2(rd.x), fast_ex2(rd.y)), Gt);
              const float2 draw = fma2(dl2, Gt, mul2(lag2, G2));
              S12 = add2(S12, u1);
              if (TRAP) {
                const float2 rawp = (k == 0) ? make_float2(prv0[e], prv0[e + 1]) : mul2(xp2, make_float2(bpv[2 * jp], bpv[2 * jp + 1]));
                S22 = fma2(aG, rawp, S22);
              }
              px2[i] = fma2(draw, b2, px2[i]);
              pB2[jp] = fma2(draw, x2, pB2[jp]);
              G[e] = aG.x; G[e + 1] = aG.y;
            }
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) px[i] = px2[i].x + px2[i].y;
#pragma unroll
          for (int jp = 0; jp < NJ / 2; ++jp) {
            pB[2 * jp] = pB2[jp].x; pB[2 * jp + 1] = pB2[jp].y;
            pC[2 * jp] = pC2[jp].x; pC[2 * jp + 1] = pC2[jp].y;
          }
          sQ = sQ2.x + sQ2.y; S1 = S12.x + S12.y; S2 = S22.x + S22.y;
          if (last) {
            // the gradient of the carried raw write joins the last token's write gradient (one token of the whole sequence)
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
              for (int jn = 0; jn < NJ; ++jn) {
                const float w = a.dwrite_last[bh * PN + (int64_t)(th.pg * 4 + i) * g.N + th.ng * NJ + jn];
                px[i] = fmaf(w, bv[jn], px[i]);
                pB[jn] = fmaf(w, xv[i], pB[jn]);
              }
          }
          lagn = dg;
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) px[i] = 0.f;
#pragma unroll
          for (int jn = 0; jn < NJ; ++jn) { pB[jn] = 0.f; pC[jn] = 0.f; }
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
        for (int i = 0; i < NJ; ++i) {
          float vb = th.active ? pB[i] : 0.f, vc = th.active ? pC[i] : 0.f;
          vb = cross_group_sum(vb, g.NG);
          vc = cross_group_sum(vc, g.NG);
          if (lane < g.NG) {
            partB[(tt * g.nwarp + warp) * g.N + lane * NJ + i] = vb;
            partC[(tt * g.nwarp + warp) * g.N + lane * NJ + i] = vc;
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
      // A warp holds 32 / NG channel groups; when NG == 32 lanes map 1:1 to row groups.  Rows n = ng * NJ + i.
      for (int idx = tid; idx < 8 * g.N; idx += blockDim.x) {
        const int tt = idx / g.N, n = idx % g.N;
        float sb = 0.f, sc = 0.f;
#pragma unroll 4
        for (int w = 0; w < g.nwarp; ++w) { sb += partB[(tt * g.nwarp + w) * g.N + n]; sc += partC[(tt * g.nwarp + w) * g.N + n]; }
        partB[(tt * g.nwarp) * g.N + n] = sb;      // slot of warp 0 now holds the total
        partC[(tt * g.nwarp) * g.N + n] = sc;
      }
      __syncthreads();
      {
        // back through the rotation: every (token, pair) is its own item; its phase gradient goes to phs / dcs
        const int lgK = 31 - __clz(g.K);
        for (int idx = tid; idx < HM_TT * g.K; idx += blockDim.x) {
          const int tt = idx >> lgK, k = idx & (g.K - 1);
          float dB = 0.f, dC = 0.f;
          if (t0 + tt < a.L && tl.rotm[k] != 0.f) {
            float2* gb = reinterpret_cast<float2*>(partB + (tt * g.nwarp) * g.N + 2 * k);
            float2* gc = reinterpret_cast<float2*>(partC + (tt * g.nwarp) * g.N + 2 * k);
            const float2 vb = *gb, vc = *gc;
            const int r = tt + 1;
            const float2 Bv = *reinterpret_cast<const float2*>(tl.Bt + r * g.N + 2 * k), Cv = *reinterpret_cast<const float2*>(tl.Ct + r * g.N + 2 * k);
            dB = vb.y * Bv.x - vb.x * Bv.y;
            dC = vc.y * Cv.x - vc.x * Cv.y;
            const float cb = tl.cB[r * g.K + k], sb = tl.sB[r * g.K + k], cc = tl.cC[r * g.K + k], sc = tl.sC[r * g.K + k];
            *gb = make_float2(vb.x * cb + vb.y * sb, -vb.x * sb + vb.y * cb);
            *gc = make_float2(vc.x * cc + vc.y * sc, -vc.x * sc + vc.y * cc);
          }
          phs[idx] = dB + dC;
          dcs[idx] = dC;
        }
      }
      __syncthreads();
      // Three independent jobs on different warps: the suffix sum of the phase gradient (first K threads, newest token
      // first), the map-gradient rows (last N threads), the drive gradient (everyone).
      if (tid < g.K) {
        const int k = tid;
        float S = Ssuf[k];
        const bool rot = tl.rotm[k] != 0.f;
#pragma unroll
        for (int tt = HM_TT - 1; tt >= 0; --tt) {
          const int tok = t0 + tt;
          if (tok >= a.L) { phs[tt * g.K + k] = 0.f; continue; }
          float ph = 0.f;
          if (rot) {
            acc_th += dcs[tt * g.K + k];
            S += phs[tt * g.K + k];
            ph = tl.featc[tt * g.K + k] * S;
          }
          if (a.dfeat_part) a.dfeat_part[(((int64_t)h * a.B + b) * a.L + tok) * g.K + k] = rot ? tl.dts[tt + 1] * S : 0.f;
          phs[tt * g.K + k] = ph;
        }
        Ssuf[k] = S;
      }
      if (tid >= (int)blockDim.x - g.N) {
        const int n = tid - ((int)blockDim.x - g.N);
        for (int tt = 0; tt < HM_TT; ++tt) {
          const int tok = t0 + tt;
          if (tok >= a.L) break;
          const float vb = partB[(tt * g.nwarp) * g.N + n], vc = partC[(tt * g.nwarp) * g.N + n];
          a.dBh_part[(((int64_t)h * a.B + b) * a.L + tok) * g.N + n] = vb;
          a.dCh_part[(((int64_t)h * a.B + b) * a.L + tok) * g.N + n] = vc;
          acc_bb += vb;
          acc_bc += vc;
        }
      }
      for (int idx = tid; idx < HM_TT * g.P; idx += blockDim.x) {
        const int tt = idx / g.P, pp = idx % g.P;
        if (t0 + tt < a.L) stf(dx + ((int64_t)b * a.L + t0 + tt) * a.H * g.P + h * g.P + pp, dxs[idx]);
      }
      if (tid < g.P)
        for (int tt = 0; tt < HM_TT; ++tt) acc_D = fmaf(tl.dys[tt * g.P + tid], tl.xs[(tt + 1) * g.P + tid], acc_D);
      __syncthreads();
      // clock gradients: one warp per token sums the per-warp partials and the phase parts (lanes take strided slices, the
      // lane sums meet in a butterfly: a fixed order)
      for (int tt = warp; tt < HM_TT; tt += g.nwarp) {
        if (t0 + tt >= a.L) continue;
        float sD = 0.f, sL = 0.f;
        for (int w = lane; w < g.nwarp; w += 32) { sD += partS[(tt * g.nwarp + w) * 2]; sL += partS[(tt * g.nwarp + w) * 2 + 1]; }
        for (int k = lane; k < g.K; k += 32) sD += phs[tt * g.K + k];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          sD += __shfl_xor_sync(0xffffffffu, sD, o);
          sL += __shfl_xor_sync(0xffffffffu, sL, o);
        }
        if (lane == 0) {
          a.ddelta[((int64_t)b * a.L + t0 + tt) * a.H + h] = sD;
          if (a.dlam) a.dlam[((int64_t)b * a.L + t0 + tt) * a.H + h] = sL;
        }
      }
      __syncthreads();
    }
  }
  // ---- what is left after token 0
  if (th.active) {
    if (a.dh_init) store_tile<NJ>(G, a.dh_init + bh * PN, th, g.N);
    if (a.dwrite_prev) {
      float wv[E];
#pragma unroll
      for (int e = 0; e < E; ++e) wv[e] = lagn * G[e];
      store_tile<NJ>(wv, a.dwrite_prev + bh * PN, th, g.N);
    }
#pragma unroll
    for (int e = 0; e < E; ++e) dA[e] *= HM_LN2;       // the sums were taken with rate2 = rate log2(e)
    store_tile<NJ>(dA, a.dA_log_part + bh * PN, th, g.N);
  }
  if (tid >= (int)blockDim.x - g.N) {
    const int n = tid - ((int)blockDim.x - g.N);
    if (a.dbeta_b_part) a.dbeta_b_part[bh * g.N + n] = acc_bb;
    if (a.dbeta_c_part) a.dbeta_c_part[bh * g.N + n] = acc_bc;
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
  {
    const HmGeo g = hm_geo(a->P, a->N);
    ORBIT_REQUIRE(g.nthr >= a->N && g.nthr >= a->P, ERR_UNSUPPORTED,
                  "%s: a CTA of (P/4)(N/4) threads, rounded up to a warp, must cover P and N (P=%d N=%d give %d threads)", who, a->P, a->N,
                  g.nthr);
  }
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

static size_t hm_smem_fwd(const HmGeo& g) { return sizeof(float) * (hm_tile_floats(g, false) + 8 * g.P + 2 * hm_raw_floats(g) + hm_plan_floats(g)); }
static size_t hm_smem_bwd(const HmGeo& g, bool keep_tiles) {
  return sizeof(float) * (hm_tile_floats(g, true, keep_tiles ? HM_SUB : 1) + (size_t)HM_SUB * g.P * g.N + r4(HM_SUB * g.K) + 2 * 8 * g.nwarp * g.N +
                          8 * g.nwarp * 2 + 8 * g.P + 2 * 8 * g.K + r4(g.K) + 32 + 2 * hm_raw_floats(g) + hm_plan_floats(g));   // (tiles: four slots)
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
  if (a->P == 64 && a->N == 64)
    rc = dtype == BF16 ? (trap ? go(hm_fwd_kernel<__nv_bfloat16, true, 64, 64>) : go(hm_fwd_kernel<__nv_bfloat16, false, 64, 64>))
                       : (trap ? go(hm_fwd_kernel<float, true, 64, 64>) : go(hm_fwd_kernel<float, false, 64, 64>));
  else
    rc = dtype == BF16 ? (trap ? go(hm_fwd_kernel<__nv_bfloat16, true, 0, 0>) : go(hm_fwd_kernel<__nv_bfloat16, false, 0, 0>))
                       : (trap ? go(hm_fwd_kernel<float, true, 0, 0>) : go(hm_fwd_kernel<float, false, 0, 0>));
  if (rc != OK) return rc;
  ORBIT_CHECK_LAUNCH("hm_fwd_kernel");
  return OK;
}

extern "C" int orbit_hm_scan_bwd(const orbit_hm_args* a, int dtype, void* stream) {
  int rc = hm_check(a, dtype, "orbit_hm_scan_bwd", true);
  if (rc != OK) return rc;
  // Four rows per thread.  Two (twice the warps at half the registers each) measured the same with compile-time geometry
  // and slower with run-time geometry (spills), so it is not instantiated.
  const HmGeo g = hm_geo(a->P, a->N, 4);
  const size_t smem = hm_smem_bwd(g, a->P == 64 && a->N == 64);
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
  if (a->P == 64 && a->N == 64)
    rc = dtype == BF16 ? (trap ? go(hm_bwd_kernel<__nv_bfloat16, true, 4, 64, 64>) : go(hm_bwd_kernel<__nv_bfloat16, false, 4, 64, 64>))
                       : (trap ? go(hm_bwd_kernel<float, true, 4, 64, 64>) : go(hm_bwd_kernel<float, false, 4, 64, 64>));
  else
    rc = dtype == BF16 ? (trap ? go(hm_bwd_kernel<__nv_bfloat16, true, 4, 0, 0>) : go(hm_bwd_kernel<__nv_bfloat16, false, 4, 0, 0>))
                       : (trap ? go(hm_bwd_kernel<float, true, 4, 0, 0>) : go(hm_bwd_kernel<float, false, 4, 0, 0>));
  if (rc != OK) return rc;
  ORBIT_CHECK_LAUNCH("hm_bwd_kernel");
  return OK;
}

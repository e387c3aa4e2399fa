// Depthwise causal conv1d (+bias, +SiLU) on token-major activations, forward and backward.
//
//   y[b,t,c] = act(bias[c] + sum_{j<W} w[c,j] * xin[b, t-(W-1)+j, c]),   xin = [carried window | x]
//
// Replaces the reference's Triton conv (src/orbit_ssm/kernels/conv_triton.py:888-1010, host entry
// src/orbit_ssm/layers/conv.py:219-328).  Layout here is token-major [B, L, C] with an arbitrary row stride, so
// the kernel reads a column slice of the fused input-projection output in place; one thread owns one 16-byte
// channel vector and slides over a run of tokens, so every warp access is a contiguous 512-byte row segment.
// HBM-bound: forward 2*B*L*C*es bytes, backward 3*B*L*C*es (x, dy in; dx out).
#include "common.cuh"
#include "../../include/orbit_b200.h"
#include <type_traits>

namespace orbit {

constexpr int CONV_MAXW = 4;
constexpr int CONV_TL = 16;   // tokens per thread run

// Raw in-flight copy of one channel vector (kept unconverted while the load is outstanding).  The vector is one
// naturally aligned load of VEC * sizeof(T) bytes: 2, 4, 8 or 16.
template <int BYTES> struct RawStore;
template <> struct RawStore<2> { using type = unsigned short; };
template <> struct RawStore<4> { using type = unsigned; };
template <> struct RawStore<8> { using type = uint2; };
template <> struct RawStore<16> { using type = uint4; };

template <typename T, int VEC>
struct RawVec {
  using Store = typename RawStore<VEC * (int)sizeof(T)>::type;
  Store r;
  __device__ __forceinline__ void load(const T* p) { r = *reinterpret_cast<const Store*>(p); }
};

template <typename T, int VEC>
struct ChanVec {
  float v[VEC];
  __device__ __forceinline__ void from_raw(const RawVec<T, VEC>& raw) {
    const T* e = reinterpret_cast<const T*>(&raw.r);
#pragma unroll
    for (int i = 0; i < VEC; ++i) v[i] = ldf(e + i);
  }
  __device__ __forceinline__ void load(const T* p) {
    RawVec<T, VEC> raw;
    raw.load(p);
    from_raw(raw);
  }
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < VEC; ++i) v[i] = 0.f;
  }
  __device__ __forceinline__ void store(T* p) const {
    typename RawVec<T, VEC>::Store r;
    T* e = reinterpret_cast<T*>(&r);
#pragma unroll
    for (int i = 0; i < VEC; ++i) stf(e + i, v[i]);
    *reinterpret_cast<typename RawVec<T, VEC>::Store*>(p) = r;
  }
};

// window: [B, C, W] fp32, slot W-1 newest; slots 1..W-1 are the W-1 raw inputs preceding this call.
template <typename T, int VEC, int W>
__device__ __forceinline__ void load_xin(ChanVec<T, VEC>& out, const T* x, int64_t xbs, int64_t xrs,
                                         const float* window, int b, int t, int c0, int C) {
  if (t >= 0) {
    out.load(x + b * xbs + (int64_t)t * xrs + c0);
  } else if (window != nullptr && t >= -(W - 1)) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) out.v[i] = window[((int64_t)b * C + c0 + i) * W + (W + t)];
  } else {
    out.zero();
  }
}

template <typename T, int VEC, int W, bool SILU>
__global__ void __launch_bounds__(128) conv_fwd_kernel(const T* __restrict__ x, int64_t xbs, int64_t xrs,
                                                       const float* __restrict__ weight,
                                                       const float* __restrict__ bias,
                                                       const float* __restrict__ window, T* __restrict__ y,
                                                       int L, int C) {
  const int c0 = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
  const int b = blockIdx.z;
  const int t0 = (blockIdx.x * blockDim.y + threadIdx.y) * CONV_TL;
  if (c0 >= C || t0 >= L) return;
  float w[VEC][W], bs[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    bs[i] = bias ? bias[c0 + i] : 0.f;
#pragma unroll
    for (int j = 0; j < W; ++j) w[i][j] = weight[(c0 + i) * W + j];
  }
  ChanVec<T, VEC> ring[W];   // ring[j] = xin[t-(W-1)+j]
#pragma unroll
  for (int j = 0; j < W - 1; ++j) load_xin<T, VEC, W>(ring[j + 1], x, xbs, xrs, window, b, t0 - (W - 1) + j, c0, C);
  const int t1 = min(t0 + CONV_TL, L);
  constexpr int NB = 8;   // rows fetched per batch: keeps NB 16-byte loads in flight per thread
  for (int tb = t0; tb < t1; tb += NB) {
    RawVec<T, VEC> in[NB];
#pragma unroll
    for (int k = 0; k < NB; ++k)
      if (tb + k < t1) in[k].load(x + b * xbs + (int64_t)(tb + k) * xrs + c0);
#pragma unroll
    for (int k = 0; k < NB; ++k) {
      if (tb + k < t1) {
#pragma unroll
        for (int j = 0; j < W - 1; ++j) ring[j] = ring[j + 1];
        ring[W - 1].from_raw(in[k]);
        ChanVec<T, VEC> o;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          float acc = bs[i];
#pragma unroll
          for (int j = 0; j < W; ++j) acc = fmaf(w[i][j], ring[j].v[i], acc);
          o.v[i] = SILU ? silu_t<T>(acc) : acc;
        }
        o.store(y + ((int64_t)b * L + tb + k) * C + c0);
      }
    }
  }
}

// Backward.  Each thread owns dx for tokens [t0, t0+TL) of its channels; it walks t up to t0+TL+W-2 so that every
// dz it needs is formed locally (pre-activations recomputed from x).  dw/db: per-thread sums over the owned tokens,
// written to `part` [(token-run index), C, W+1] and reduced in a fixed order by conv_reduce_kernel (deterministic).
template <typename T, int VEC, int W, bool SILU>
__global__ void __launch_bounds__(128) conv_bwd_kernel(const T* __restrict__ x, int64_t xbs, int64_t xrs,
                                                       const float* __restrict__ weight,
                                                       const float* __restrict__ bias,
                                                       const float* __restrict__ window,
                                                       const T* __restrict__ dy, T* __restrict__ dx, int64_t dxbs,
                                                       int64_t dxrs, float* __restrict__ dwindow,
                                                       float* __restrict__ part, int L, int C, int nruns) {
  const int c0 = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
  const int b = blockIdx.z;
  const int run = blockIdx.x * blockDim.y + threadIdx.y;
  const int t0 = run * CONV_TL;
  if (c0 >= C || t0 >= L) return;
  float w[VEC][W], bs[VEC], dwacc[VEC][W], dbacc[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    bs[i] = bias ? bias[c0 + i] : 0.f;
    dbacc[i] = 0.f;
#pragma unroll
    for (int j = 0; j < W; ++j) {
      w[i][j] = weight[(c0 + i) * W + j];
      dwacc[i][j] = 0.f;
    }
  }
  ChanVec<T, VEC> ring[W];      // xin[t-(W-1)+j]
  float dz[W][VEC];             // dz[k] = dz at token t-k
#pragma unroll
  for (int k = 0; k < W; ++k)
#pragma unroll
    for (int i = 0; i < VEC; ++i) dz[k][i] = 0.f;
#pragma unroll
  for (int j = 0; j < W - 1; ++j) load_xin<T, VEC, W>(ring[j + 1], x, xbs, xrs, window, b, t0 - (W - 1) + j, c0, C);
  const int t_own_end = min(t0 + CONV_TL, L);
  const int t_end = min(t0 + CONV_TL + W - 1, L + W - 1);   // walk far enough to emit dx of the last owned token
  constexpr int NB = 4;   // rows of x and dy fetched per batch
  for (int tb = t0; tb < t_end; tb += NB) {
    RawVec<T, VEC> xin[NB], gin[NB];
#pragma unroll
    for (int k = 0; k < NB; ++k)
      if (tb + k < t_end && tb + k < L) {
        xin[k].load(x + b * xbs + (int64_t)(tb + k) * xrs + c0);
        gin[k].load(dy + ((int64_t)b * L + tb + k) * C + c0);
      }
#pragma unroll
    for (int kk = 0; kk < NB; ++kk) {
      const int t = tb + kk;
      if (t >= t_end) break;
#pragma unroll
      for (int k = W - 1; k > 0; --k)
#pragma unroll
        for (int i = 0; i < VEC; ++i) dz[k][i] = dz[k - 1][i];
      if (t < L) {
#pragma unroll
        for (int j = 0; j < W - 1; ++j) ring[j] = ring[j + 1];
        ring[W - 1].from_raw(xin[kk]);
        ChanVec<T, VEC> gv;
        gv.from_raw(gin[kk]);
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          float pre = bs[i];
#pragma unroll
          for (int j = 0; j < W; ++j) pre = fmaf(w[i][j], ring[j].v[i], pre);
          float d = SILU ? gv.v[i] * silu_grad_t<T>(pre) : gv.v[i];
          dz[0][i] = d;
          if (t < t_own_end) {
            dbacc[i] += d;
#pragma unroll
            for (int j = 0; j < W; ++j) dwacc[i][j] = fmaf(d, ring[j].v[i], dwacc[i][j]);
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) dz[0][i] = 0.f;
      }
      // dx[t'] with t' = t-(W-1):  sum_j w[j] dz[t'+(W-1)-j] = sum_j w[j] dz_at(t-j)
      const int tp = t - (W - 1);
      if (tp >= t0 || (t0 == 0 && dwindow != nullptr)) {
        ChanVec<T, VEC> o;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          float acc = 0.f;
#pragma unroll
          for (int j = 0; j < W; ++j) acc = fmaf(w[i][j], dz[j][i], acc);
          o.v[i] = acc;
        }
        if (tp >= t0) {
          if (tp < t_own_end) o.store(dx + b * dxbs + (int64_t)tp * dxrs + c0);
        } else if (tp >= -(W - 1)) {   // gradient of the carried window (slots 1..W-1)
#pragma unroll
          for (int i = 0; i < VEC; ++i) dwindow[((int64_t)b * C + c0 + i) * W + (W + tp)] = o.v[i];
        }
      }
    }
  }
  if (part != nullptr) {
    float* p = part + ((int64_t)(b * nruns + run) * C + c0) * (W + 1);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
#pragma unroll
      for (int j = 0; j < W; ++j) p[i * (W + 1) + j] = dwacc[i][j];
      p[i * (W + 1) + W] = dbacc[i];
    }
  }
}

// ---- shared-memory tiled variants (the fast path) ---------------------------------------------------------------------
// A CTA stages a [TT + halo tokens] x [32 channel vectors] tile with every 16-byte load in flight at once, then warp w
// slides over tokens 8w..8w+7 of the tile with lane = channel vector.  Rows before the sequence start come from the
// carried window (or zeros).  Used when C is a multiple of 32 vectors and no window gradient is asked for.
constexpr int CT_TT = 64;        // tokens per tile
constexpr int CT_WARPS = 8;      // 8 tokens per warp

template <typename T, int VEC, int W>
__device__ __forceinline__ void tile_row(RawVec<T, VEC>& out, const T* x, int64_t xbs, int64_t xrs, const float* window,
                                         int b, int t, int L, int c0, int C) {
  if (t >= 0 && t < L) {
    out.load(x + b * xbs + (int64_t)t * xrs + c0);
  } else {
    T tmp[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      float v = 0.f;
      if (t < 0 && window != nullptr && t >= -(W - 1)) v = window[((int64_t)b * C + c0 + i) * W + (W + t)];
      stf(&tmp[i], v);
    }
    out.r = *reinterpret_cast<const typename RawVec<T, VEC>::Store*>(tmp);
  }
}

// taps and bias of VEC consecutive channels (one 16-byte load per channel when W == 4)
template <int VEC, int W>
__device__ __forceinline__ void load_taps(float (&w)[VEC][W], float (&bs)[VEC], const float* __restrict__ weight,
                                          const float* __restrict__ bias, int c0) {
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    if constexpr (W == 4) {
      float4 v = *reinterpret_cast<const float4*>(weight + (size_t)(c0 + i) * 4);
      w[i][0] = v.x; w[i][1] = v.y; w[i][2] = v.z; w[i][3] = v.w;
    } else {
#pragma unroll
      for (int j = 0; j < W; ++j) w[i][j] = weight[(c0 + i) * W + j];
    }
    bs[i] = bias ? bias[c0 + i] : 0.f;
  }
}

constexpr int CT_NT = 4;         // consecutive token tiles per CTA (taps stay in registers across them)

template <typename T, int VEC, int W, bool SILU>
__global__ void __launch_bounds__(256, (VEC * sizeof(T) >= 16) ? 2 : 4) conv_fwd_tiled_kernel(const T* __restrict__ x, int64_t xbs, int64_t xrs,
                                                             const float* __restrict__ weight, const float* __restrict__ bias,
                                                             const float* __restrict__ window, T* __restrict__ y, int L, int C) {
  __shared__ RawVec<T, VEC> tile[CT_TT + W - 1][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = (blockIdx.y * 32 + lane) * VEC;
  const int b = blockIdx.z;
  float w[VEC][W], bs[VEC];
  load_taps<VEC, W>(w, bs, weight, bias, c0);
  for (int it = 0; it < CT_NT; ++it) {
    const int t0 = (blockIdx.x * CT_NT + it) * CT_TT;
    if (t0 >= L) break;
    __syncthreads();
    for (int r = warp; r < CT_TT + W - 1; r += CT_WARPS) tile_row<T, VEC, W>(tile[r][lane], x, xbs, xrs, window, b, t0 - (W - 1) + r, L, c0, C);
    __syncthreads();
    const int tw = warp * (CT_TT / CT_WARPS);
    ChanVec<T, VEC> ring[W];
#pragma unroll
    for (int j = 0; j < W - 1; ++j) ring[j + 1].from_raw(tile[tw + j][lane]);
#pragma unroll
    for (int k = 0; k < CT_TT / CT_WARPS; ++k) {
      const int t = t0 + tw + k;
#pragma unroll
      for (int j = 0; j < W - 1; ++j) ring[j] = ring[j + 1];
      ring[W - 1].from_raw(tile[tw + k + W - 1][lane]);
      if (t < L) {
        ChanVec<T, VEC> o;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          float acc = bs[i];
#pragma unroll
          for (int j = 0; j < W; ++j) acc = fmaf(w[i][j], ring[j].v[i], acc);
          o.v[i] = SILU ? silu_t<T>(acc) : acc;
        }
        o.store(y + ((int64_t)b * L + t) * C + c0);
      }
    }
  }
}

// Backward, tiled.  Warp w owns dx (and the dw/db contributions) of tokens 8w..8w+7; it forms dz for 8 + (W-1) tokens.
// dw/db: per-thread sums -> shared [warp][lane] -> fixed-order sum over the 8 warps -> part[(b, tile)][C][W+1].
constexpr int CTB_TT = 32;       // backward: tokens per tile
constexpr int CTB_WARPS = 4;

template <typename T, int VEC, int W, bool SILU>
__global__ void __launch_bounds__(CTB_WARPS * 32, (VEC * sizeof(T) >= 16) ? 2 : 4) conv_bwd_tiled_kernel(const T* __restrict__ x, int64_t xbs, int64_t xrs,
                                                             const float* __restrict__ weight, const float* __restrict__ bias,
                                                             const float* __restrict__ window, const T* __restrict__ dy,
                                                             T* __restrict__ dx, int64_t dxbs, int64_t dxrs,
                                                             float* __restrict__ part, int L, int C, int ntiles) {
  constexpr int TW = CTB_TT / CTB_WARPS;
  constexpr int XR = CTB_TT + 2 * (W - 1), GR = CTB_TT + W - 1, RED_E = VEC * (W + 1) + 1;
  constexpr size_t TILE_BYTES = sizeof(RawVec<T, VEC>) * 32 * (XR + GR), RED_BYTES = sizeof(float) * CTB_WARPS * 32 * RED_E;
  __shared__ __align__(16) unsigned char sraw[TILE_BYTES > RED_BYTES ? TILE_BYTES : RED_BYTES];
  RawVec<T, VEC>(*xt)[32] = reinterpret_cast<RawVec<T, VEC>(*)[32]>(sraw);                                 // x rows t0-(W-1) ..
  RawVec<T, VEC>(*gt)[32] = reinterpret_cast<RawVec<T, VEC>(*)[32]>(sraw + sizeof(RawVec<T, VEC>) * 32 * XR);  // dy rows t0 ..
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = (blockIdx.y * 32 + lane) * VEC;
  const int b = blockIdx.z;
  float w[VEC][W], bs[VEC], dwacc[VEC][W], dbacc[VEC];
  load_taps<VEC, W>(w, bs, weight, bias, c0);
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    dbacc[i] = 0.f;
#pragma unroll
    for (int j = 0; j < W; ++j) dwacc[i][j] = 0.f;
  }
  for (int it = 0; it < CT_NT; ++it) {
    const int t0 = (blockIdx.x * CT_NT + it) * CTB_TT;
    if (t0 >= L) break;
    __syncthreads();
    for (int r = warp; r < XR; r += CTB_WARPS) tile_row<T, VEC, W>(xt[r][lane], x, xbs, xrs, window, b, t0 - (W - 1) + r, L, c0, C);
    for (int r = warp; r < GR; r += CTB_WARPS) tile_row<T, VEC, W>(gt[r][lane], dy, (int64_t)L * C, C, nullptr, b, (t0 + r < L) ? t0 + r : -W, L, c0, C);
    __syncthreads();
    const int tw = warp * TW;
    ChanVec<T, VEC> ring[W];
    float dz[W][VEC];
#pragma unroll
    for (int k = 0; k < W; ++k)
#pragma unroll
      for (int i = 0; i < VEC; ++i) dz[k][i] = 0.f;
#pragma unroll
    for (int j = 0; j < W - 1; ++j) ring[j + 1].from_raw(xt[tw + j][lane]);      // x rows (t0+tw)-(W-1) ..
#pragma unroll
    for (int k = 0; k < TW + W - 1; ++k) {
      const int t = t0 + tw + k;
#pragma unroll
      for (int kk = W - 1; kk > 0; --kk)
#pragma unroll
        for (int i = 0; i < VEC; ++i) dz[kk][i] = dz[kk - 1][i];
#pragma unroll
      for (int j = 0; j < W - 1; ++j) ring[j] = ring[j + 1];
      ring[W - 1].from_raw(xt[tw + k + W - 1][lane]);
      ChanVec<T, VEC> gv;
      gv.from_raw(gt[tw + k][lane]);                    // zero past the sequence end
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        float pre = bs[i];
#pragma unroll
        for (int j = 0; j < W; ++j) pre = fmaf(w[i][j], ring[j].v[i], pre);
        float d = SILU ? gv.v[i] * silu_grad_t<T>(pre) : gv.v[i];
        dz[0][i] = d;
        if (k < TW) {
          dbacc[i] += d;
#pragma unroll
          for (int j = 0; j < W; ++j) dwacc[i][j] = fmaf(d, ring[j].v[i], dwacc[i][j]);
        }
      }
      if (k >= W - 1) {
        const int tp = t - (W - 1);
        if (tp < L) {
          ChanVec<T, VEC> o;
#pragma unroll
          for (int i = 0; i < VEC; ++i) {
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < W; ++j) acc = fmaf(w[i][j], dz[j][i], acc);
            o.v[i] = acc;
          }
          o.store(dx + b * dxbs + (int64_t)tp * dxrs + c0);
        }
      }
    }
  }
  if (part != nullptr) {
    __syncthreads();                                   // the tiles are dead: their storage becomes the reduction buffer
    float(*red)[32][RED_E] = reinterpret_cast<float(*)[32][RED_E]>(sraw);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
#pragma unroll
      for (int j = 0; j < W; ++j) red[warp][lane][i * (W + 1) + j] = dwacc[i][j];
      red[warp][lane][i * (W + 1) + W] = dbacc[i];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < 32 * VEC * (W + 1); idx += CTB_WARPS * 32) {
      const int l = idx / (VEC * (W + 1)), e = idx % (VEC * (W + 1));
      float acc = 0.f;
#pragma unroll
      for (int ww = 0; ww < CTB_WARPS; ++ww) acc += red[ww][l][e];
      part[((int64_t)(b * ntiles + blockIdx.x) * C + (blockIdx.y * 32 + l) * VEC) * (W + 1) + e] = acc;
    }
  }
}

// out[c, k] = sum over partial slots (fixed order), k < W -> dweight[c,k], k == W -> dbias[c]
__global__ void conv_reduce_kernel(const float* __restrict__ part, float* __restrict__ dweight,
                                   float* __restrict__ dbias, int nslots, int C, int W) {
  int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= C * (W + 1)) return;
  float acc = 0.f;
  for (int s = 0; s < nslots; ++s) acc += part[(int64_t)s * C * (W + 1) + idx];
  int c = idx / (W + 1), k = idx % (W + 1);
  if (k < W) dweight[c * W + k] = acc;
  else if (dbias) dbias[c] = acc;
}

static inline void conv_grid(int B, int L, int C, int VEC, dim3& grid, dim3& block) {
  int cv = (C + VEC - 1) / VEC;
  int bx = cv >= 128 ? 128 : (cv >= 64 ? 64 : 32);
  int by = 128 / bx;
  int runs = (L + CONV_TL - 1) / CONV_TL;
  block = dim3(bx, by, 1);
  grid = dim3((runs + by - 1) / by, (cv + bx - 1) / bx, B);
}

template <typename T, int VEC, int W>
static int conv_fwd_launch(const T* x, int64_t xbs, int64_t xrs, const float* w, const float* b, const float* win,
                           T* y, int B, int L, int C, int silu, cudaStream_t st) {
  if (VEC > 1 && C % (32 * VEC) == 0) {
    dim3 tg((L + CT_TT * CT_NT - 1) / (CT_TT * CT_NT), C / (32 * VEC), B);
    if (silu) conv_fwd_tiled_kernel<T, VEC, W, true><<<tg, 256, 0, st>>>(x, xbs, xrs, w, b, win, y, L, C);
    else conv_fwd_tiled_kernel<T, VEC, W, false><<<tg, 256, 0, st>>>(x, xbs, xrs, w, b, win, y, L, C);
    ORBIT_CHECK_LAUNCH("conv_fwd_tiled_kernel");
    return OK;
  }
  dim3 grid, block;
  conv_grid(B, L, C, VEC, grid, block);
  if (silu) conv_fwd_kernel<T, VEC, W, true><<<grid, block, 0, st>>>(x, xbs, xrs, w, b, win, y, L, C);
  else conv_fwd_kernel<T, VEC, W, false><<<grid, block, 0, st>>>(x, xbs, xrs, w, b, win, y, L, C);
  ORBIT_CHECK_LAUNCH("conv_fwd_kernel");
  return OK;
}

template <typename T, int VEC, int W>
static int conv_bwd_launch(const T* x, int64_t xbs, int64_t xrs, const float* w, const float* b, const float* win,
                           const T* dy, T* dx, int64_t dxbs, int64_t dxrs, float* dwin, float* part, int B, int L,
                           int C, int silu, cudaStream_t st, int* nslots) {
  *nslots = B * ((L + CONV_TL - 1) / CONV_TL);
  if (VEC > 1 && C % (32 * VEC) == 0 && dwin == nullptr) {
    const int ntiles = (L + CTB_TT * CT_NT - 1) / (CTB_TT * CT_NT);
    *nslots = B * ntiles;
    dim3 tg(ntiles, C / (32 * VEC), B);
    if (silu) conv_bwd_tiled_kernel<T, VEC, W, true><<<tg, CTB_WARPS * 32, 0, st>>>(x, xbs, xrs, w, b, win, dy, dx, dxbs, dxrs, part, L, C, ntiles);
    else conv_bwd_tiled_kernel<T, VEC, W, false><<<tg, CTB_WARPS * 32, 0, st>>>(x, xbs, xrs, w, b, win, dy, dx, dxbs, dxrs, part, L, C, ntiles);
    ORBIT_CHECK_LAUNCH("conv_bwd_tiled_kernel");
    return OK;
  }
  dim3 grid, block;
  conv_grid(B, L, C, VEC, grid, block);
  int nruns = (L + CONV_TL - 1) / CONV_TL;
  if (silu)
    conv_bwd_kernel<T, VEC, W, true><<<grid, block, 0, st>>>(x, xbs, xrs, w, b, win, dy, dx, dxbs, dxrs, dwin, part,
                                                             L, C, nruns);
  else
    conv_bwd_kernel<T, VEC, W, false><<<grid, block, 0, st>>>(x, xbs, xrs, w, b, win, dy, dx, dxbs, dxrs, dwin,
                                                              part, L, C, nruns);
  ORBIT_CHECK_LAUNCH("conv_bwd_kernel");
  return OK;
}

template <typename T>
static bool conv_vec_ok(const void* x, int64_t xbs, int64_t xrs, const void* y, int C, const void* p2 = nullptr,
                        int64_t s2a = 0, int64_t s2b = 0) {
  constexpr int V = Vec16<T>::N;
  return C % V == 0 && xbs % V == 0 && xrs % V == 0 && aligned16(x) && aligned16(y) && s2a % V == 0 && s2b % V == 0 &&
         (p2 == nullptr || aligned16(p2));
}

}  // namespace orbit

using namespace orbit;

#define CONV_DISPATCH_W(FN, T, VEC, ...)                                                 \
  switch (W) {                                                                           \
    case 2: return FN<T, VEC, 2>(__VA_ARGS__);                                           \
    case 3: return FN<T, VEC, 3>(__VA_ARGS__);                                           \
    case 4: return FN<T, VEC, 4>(__VA_ARGS__);                                           \
    default: return fail(ERR_UNSUPPORTED, "conv width W=%d: kernel serves 2..4", W);     \
  }

extern "C" int64_t orbit_conv1d_bwd_workspace_bytes(int B, int L, int C, int W) {
  int64_t nruns = (L + CONV_TL - 1) / CONV_TL;
  return (int64_t)B * nruns * C * (W + 1) * (int64_t)sizeof(float);
}

extern "C" int orbit_conv1d_fwd(const void* x, int64_t x_batch_stride, int64_t x_row_stride, const float* weight,
                                const float* bias, const float* window, void* y, int B, int L, int C, int W,
                                int dtype, int silu, void* stream) {
  ORBIT_REQUIRE(x && weight && y, ERR_BAD_ARG, "orbit_conv1d_fwd: null x/weight/y");
  ORBIT_REQUIRE(B >= 0 && L >= 0 && C > 0, ERR_BAD_ARG, "orbit_conv1d_fwd: bad sizes B=%d L=%d C=%d", B, L, C);
  if (B == 0 || L == 0) return OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == BF16) {
    using T = __nv_bfloat16;
    if (conv_vec_ok<T>(x, x_batch_stride, x_row_stride, y, C)) {
      if (C % 128 == 0) {   // tiled path: 8-byte vectors keep 32 warps resident per SM
        CONV_DISPATCH_W(conv_fwd_launch, T, 4, (const T*)x, x_batch_stride, x_row_stride, weight, bias, window, (T*)y, B,
                        L, C, silu, st)
      }
      CONV_DISPATCH_W(conv_fwd_launch, T, 8, (const T*)x, x_batch_stride, x_row_stride, weight, bias, window, (T*)y, B,
                      L, C, silu, st)
    }
    CONV_DISPATCH_W(conv_fwd_launch, T, 1, (const T*)x, x_batch_stride, x_row_stride, weight, bias, window, (T*)y, B, L,
                    C, silu, st)
  } else if (dtype == F32) {
    using T = float;
    if (conv_vec_ok<T>(x, x_batch_stride, x_row_stride, y, C)) {
      CONV_DISPATCH_W(conv_fwd_launch, T, 4, (const T*)x, x_batch_stride, x_row_stride, weight, bias, window, (T*)y, B,
                      L, C, silu, st)
    }
    CONV_DISPATCH_W(conv_fwd_launch, T, 1, (const T*)x, x_batch_stride, x_row_stride, weight, bias, window, (T*)y, B, L,
                    C, silu, st)
  }
  return fail(ERR_BAD_ARG, "orbit_conv1d_fwd: unknown dtype code %d", dtype);
}

extern "C" int orbit_conv1d_bwd(const void* x, int64_t x_batch_stride, int64_t x_row_stride, const float* weight,
                                const float* bias, const float* window, const void* dy, void* dx,
                                int64_t dx_batch_stride, int64_t dx_row_stride, float* dwindow, float* dweight,
                                float* dbias, void* workspace, int64_t workspace_bytes, int B, int L, int C, int W,
                                int dtype, int silu, void* stream) {
  ORBIT_REQUIRE(x && weight && dy && dx, ERR_BAD_ARG, "orbit_conv1d_bwd: null x/weight/dy/dx");
  ORBIT_REQUIRE(B >= 0 && L >= 0 && C > 0, ERR_BAD_ARG, "orbit_conv1d_bwd: bad sizes B=%d L=%d C=%d", B, L, C);
  ORBIT_REQUIRE(W >= 2 && W <= CONV_MAXW, ERR_UNSUPPORTED, "conv width W=%d: kernel serves 2..4", W);
  cudaStream_t st = (cudaStream_t)stream;
  if (B == 0 || L == 0) {
    if (dweight) ORBIT_CHECK_CUDA(cudaMemsetAsync(dweight, 0, sizeof(float) * C * W, st));
    if (dbias) ORBIT_CHECK_CUDA(cudaMemsetAsync(dbias, 0, sizeof(float) * C, st));
    if (dwindow) ORBIT_CHECK_CUDA(cudaMemsetAsync(dwindow, 0, sizeof(float) * (size_t)B * C * W, st));
    return OK;
  }
  float* part = nullptr;
  if (dweight) {
    ORBIT_REQUIRE(workspace && workspace_bytes >= orbit_conv1d_bwd_workspace_bytes(B, L, C, W), ERR_WORKSPACE,
                  "orbit_conv1d_bwd: workspace of %lld bytes needed", (long long)orbit_conv1d_bwd_workspace_bytes(B, L, C, W));
    part = (float*)workspace;
  }
  if (dwindow) ORBIT_CHECK_CUDA(cudaMemsetAsync(dwindow, 0, sizeof(float) * (size_t)B * C * W, st));
  int rc = -1, nslots = 0;
  auto go = [&]() -> int {
    if (dtype == BF16) {
      using T = __nv_bfloat16;
      if (conv_vec_ok<T>(x, x_batch_stride, x_row_stride, dy, C, dx, dx_batch_stride, dx_row_stride)) {
        if (C % 128 == 0 && dwindow == nullptr) {   // tiled path: 8-byte vectors keep 16 warps resident per SM
          CONV_DISPATCH_W(conv_bwd_launch, T, 4, (const T*)x, x_batch_stride, x_row_stride, weight, bias, window,
                          (const T*)dy, (T*)dx, dx_batch_stride, dx_row_stride, dwindow, part, B, L, C, silu, st, &nslots)
        }
        CONV_DISPATCH_W(conv_bwd_launch, T, 8, (const T*)x, x_batch_stride, x_row_stride, weight, bias, window,
                        (const T*)dy, (T*)dx, dx_batch_stride, dx_row_stride, dwindow, part, B, L, C, silu, st, &nslots)
      }
      CONV_DISPATCH_W(conv_bwd_launch, T, 1, (const T*)x, x_batch_stride, x_row_stride, weight, bias, window,
                      (const T*)dy, (T*)dx, dx_batch_stride, dx_row_stride, dwindow, part, B, L, C, silu, st, &nslots)
    } else if (dtype == F32) {
      using T = float;
      if (conv_vec_ok<T>(x, x_batch_stride, x_row_stride, dy, C, dx, dx_batch_stride, dx_row_stride)) {
        CONV_DISPATCH_W(conv_bwd_launch, T, 4, (const T*)x, x_batch_stride, x_row_stride, weight, bias, window,
                        (const T*)dy, (T*)dx, dx_batch_stride, dx_row_stride, dwindow, part, B, L, C, silu, st, &nslots)
      }
      CONV_DISPATCH_W(conv_bwd_launch, T, 1, (const T*)x, x_batch_stride, x_row_stride, weight, bias, window,
                      (const T*)dy, (T*)dx, dx_batch_stride, dx_row_stride, dwindow, part, B, L, C, silu, st, &nslots)
    }
    return fail(ERR_BAD_ARG, "orbit_conv1d_bwd: unknown dtype code %d", dtype);
  };
  rc = go();
  if (rc != OK) return rc;
  if (dweight) {
    int n = C * (W + 1);
    conv_reduce_kernel<<<(n + 255) / 256, 256, 0, st>>>(part, dweight, dbias, nslots, C, W);
    ORBIT_CHECK_LAUNCH("conv_reduce_kernel");
  }
  return OK;
}

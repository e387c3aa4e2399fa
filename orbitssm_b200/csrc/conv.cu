// Depthwise causal conv1d (+bias, +SiLU) on token-major activations, forward and backward.
//
//   y[b,t,c] = act(bias[c] + sum_{j<W} w[c,j] * xin[b, t-(W-1)+j, c]),   xin = [carried window | x]
//
// Replaces the reference's Triton conv (src/orbit_ssm/kernels/conv_triton.py:888-1010, host entry
// src/orbit_ssm/layers/conv.py:219-328).  Layout here is token-major [B, L, C] with an arbitrary row stride, so
// the kernel reads a column slice of the fused input-projection output in place; one thread owns one channel
// vector and slides over a run of tokens, so every warp access is a contiguous row segment.
// HBM-bound: forward 2*B*L*C*es bytes, backward 3*B*L*C*es (x, dy in; dx out).  Channel counts that fill whole warps
// with 4-channel vectors take the streaming kernels (cp.async rings, packed fp32 pairs); the rest take the plain
// per-thread kernels above them.
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

// ---- streaming variants (the fast path) -------------------------------------------------------------------------------
// A thread owns one channel vector (8 or 16 bytes of consecutive channels) and walks a run of consecutive tokens.  Its
// rows arrive through a private ring of cp.async stages in shared memory (CS_ROWS rows per stage, CS_STAGES stages), so
// loads of the rows ahead are in flight while the current rows are computed and no thread waits on another: the kernel
// has no barrier.  A CTA is `cx` channel vectors wide (a warp reads one contiguous 256- or 512-byte segment per row) and
// 128 / cx token runs deep.  Arithmetic is on packed fp32 pairs; rows before the sequence start come from the carried
// window (or zeros) and are written to the ring by the thread itself.
constexpr int CS_THREADS = 128;
constexpr int CS_ROWS = 4;
constexpr int CS_STAGES = 4;

template <int BYTES> __device__ __forceinline__ void cs_copy(void* smem_dst, const void* gsrc);
template <> __device__ __forceinline__ void cs_copy<16>(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}
template <> __device__ __forceinline__ void cs_copy<8>(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cs_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cs_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// channel vector <-> packed fp32 pairs
template <typename T, int VEC> struct Pairs {
  using Raw = typename RawStore<VEC * (int)sizeof(T)>::type;
  float2 p[VEC / 2];
  __device__ __forceinline__ void from_raw(const Raw& r) {
    if constexpr (std::is_same<T, float>::value) {
      const float* f = reinterpret_cast<const float*>(&r);
#pragma unroll
      for (int i = 0; i < VEC / 2; ++i) p[i] = make_float2(f[2 * i], f[2 * i + 1]);
    } else {
      const uint32_t* u = reinterpret_cast<const uint32_t*>(&r);
#pragma unroll
      for (int i = 0; i < VEC / 2; ++i) p[i] = make_float2(__uint_as_float(u[i] << 16), __uint_as_float(u[i] & 0xffff0000u));
    }
  }
  __device__ __forceinline__ Raw to_raw() const {
    Raw r;
    if constexpr (std::is_same<T, float>::value) {
      float* f = reinterpret_cast<float*>(&r);
#pragma unroll
      for (int i = 0; i < VEC / 2; ++i) { f[2 * i] = p[i].x; f[2 * i + 1] = p[i].y; }
    } else {
      uint32_t* u = reinterpret_cast<uint32_t*>(&r);
#pragma unroll
      for (int i = 0; i < VEC / 2; ++i) u[i] = pack_bf16(p[i].x, p[i].y);
    }
    return r;
  }
};

// silu(v) and d silu / dv on a pair: bfloat16 activations take the single-MUFU tanh form (as Act<__nv_bfloat16>)
template <typename T> __device__ __forceinline__ float2 silu2(float2 v) {
  if constexpr (std::is_same<T, float>::value) {
    return make_float2(silu_t<float>(v.x), silu_t<float>(v.y));
  } else {
    const float2 h = mul2(v, make_float2(0.5f, 0.5f));
    const float2 th = make_float2(tanh_approx_(h.x), tanh_approx_(h.y));
    return fma2(h, th, h);
  }
}
template <typename T> __device__ __forceinline__ float2 silu_grad2(float2 v) {
  if constexpr (std::is_same<T, float>::value) {
    return make_float2(silu_grad_t<float>(v.x), silu_grad_t<float>(v.y));
  } else {
    const float2 half = make_float2(0.5f, 0.5f), one = make_float2(1.f, 1.f);
    const float2 h = mul2(v, half);
    const float2 th = make_float2(tanh_approx_(h.x), tanh_approx_(h.y));
    const float2 s = fma2(half, th, half);
    const float2 om = fma2(s, make_float2(-1.f, -1.f), one);
    return mul2(s, fma2(v, om, one));
  }
}

template <int VEC, int W>
__device__ __forceinline__ void load_taps2(float2 (&w2)[W][VEC / 2], float2 (&b2)[VEC / 2], const float* __restrict__ weight,
                                           const float* __restrict__ bias, int c0) {
#pragma unroll
  for (int i = 0; i < VEC / 2; ++i) {
#pragma unroll
    for (int j = 0; j < W; ++j) w2[j][i] = make_float2(weight[(size_t)(c0 + 2 * i) * W + j], weight[(size_t)(c0 + 2 * i + 1) * W + j]);
    b2[i] = bias ? make_float2(bias[c0 + 2 * i], bias[c0 + 2 * i + 1]) : make_float2(0.f, 0.f);
  }
}

// row of the carried window (token t < 0) as a raw channel vector
template <typename T, int VEC, int W>
__device__ __forceinline__ typename Pairs<T, VEC>::Raw window_row(const float* __restrict__ window, int b, int t, int c0, int C) {
  T tmp[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    float v = 0.f;
    if (window != nullptr && t >= -(W - 1)) v = window[((int64_t)b * C + c0 + i) * W + (W + t)];
    stf(&tmp[i], v);
  }
  return *reinterpret_cast<const typename Pairs<T, VEC>::Raw*>(tmp);
}

template <typename T, int VEC, int W, bool SILU>
__global__ void __launch_bounds__(CS_THREADS) conv_fwd_stream_kernel(const T* __restrict__ x, int64_t xbs, int64_t xrs,
                                                                     const float* __restrict__ weight, const float* __restrict__ bias,
                                                                     const float* __restrict__ window, T* __restrict__ y, int L, int C,
                                                                     int run, int cx) {
  using P = Pairs<T, VEC>;
  using Raw = typename P::Raw;
  constexpr int BYTES = VEC * (int)sizeof(T);
  __shared__ Raw ring[CS_STAGES][CS_ROWS][CS_THREADS];
  const int tid = threadIdx.x;
  const int c0 = (blockIdx.y * cx + (tid & (cx - 1))) * VEC;
  const int b = blockIdx.z;
  const int t0 = (blockIdx.x * (CS_THREADS / cx) + tid / cx) * run;
  if (t0 >= L) return;
  const int ntok = min(run, L - t0);
  const int nrows = ntok + W - 1;                       // row i <-> token t0 - (W-1) + i
  const int nst = (nrows + CS_ROWS - 1) / CS_ROWS;
  const T* xb = x + b * xbs + c0;
  auto issue = [&](int s) {
    if (s < nst) {
#pragma unroll
      for (int r = 0; r < CS_ROWS; ++r) {
        const int i = s * CS_ROWS + r, t = t0 - (W - 1) + i;
        Raw* dst = &ring[s & (CS_STAGES - 1)][r][tid];
        if (i < nrows) {
          if (t >= 0) cs_copy<BYTES>(dst, xb + (int64_t)t * xrs);
          else *dst = window_row<T, VEC, W>(window, b, t, c0, C);
        }
      }
    }
    cs_commit();
  };
  float2 w2[W][VEC / 2], b2[VEC / 2];
#pragma unroll
  for (int s = 0; s < CS_STAGES - 1; ++s) issue(s);
  load_taps2<VEC, W>(w2, b2, weight, bias, c0);
  P xr[W];                                              // xr[j] = input row of token t - (W-1) + j
#pragma unroll
  for (int j = 0; j < W; ++j)
#pragma unroll
    for (int i = 0; i < VEC / 2; ++i) xr[j].p[i] = make_float2(0.f, 0.f);
  T* yb = y + ((int64_t)b * L + t0) * C + c0;
  // one row of the walk; FULL: the row is known to be inside the run and past the halo (no tests, so that the rows of a
  // stage form one straight-line block the compiler can interleave)
  auto row = [&](int s, int r, auto full) {
    constexpr bool FULL = decltype(full)::value;
    const int i = s * CS_ROWS + r;
    if (FULL || i < nrows) {
      const Raw raw = ring[s & (CS_STAGES - 1)][r][tid];
#pragma unroll
      for (int j = 0; j < W - 1; ++j) xr[j] = xr[j + 1];
      xr[W - 1].from_raw(raw);
      if (FULL || i >= W - 1) {
        P o;
#pragma unroll
        for (int k = 0; k < VEC / 2; ++k) {
          float2 acc = b2[k];
#pragma unroll
          for (int j = 0; j < W; ++j) acc = fma2(w2[j][k], xr[j].p[k], acc);
          o.p[k] = SILU ? silu2<T>(acc) : acc;
        }
        *reinterpret_cast<Raw*>(yb + (int64_t)(i - (W - 1)) * C) = o.to_raw();
      }
    }
  };
  for (int s = 0; s < nst; ++s) {
    issue(s + CS_STAGES - 1);
    cs_wait<CS_STAGES - 1>();
    if (s >= 1 && s * CS_ROWS + CS_ROWS <= nrows) {
#pragma unroll
      for (int r = 0; r < CS_ROWS; ++r) row(s, r, std::true_type{});
    } else {
#pragma unroll
      for (int r = 0; r < CS_ROWS; ++r) row(s, r, std::false_type{});
    }
  }
}

// Backward, streaming.  A thread owns dx (and the dw / db contributions) of the tokens of its run; it forms dz for W - 1
// more tokens past the run so that every dx it owns is complete (pre-activations recomputed from x).  Row i of its walk
// is token t0 - (W-1) + i: x rows from i = 0, dy rows from i = W - 1, dx rows leave from i = 2 (W - 1).  dw / db: per-thread
// sums over the owned tokens -> part[(b, run)][C][W + 1], reduced in a fixed order by conv_reduce_kernel.
template <typename T, int VEC, int W, bool SILU>
__global__ void __launch_bounds__(CS_THREADS) conv_bwd_stream_kernel(const T* __restrict__ x, int64_t xbs, int64_t xrs,
                                                                     const float* __restrict__ weight, const float* __restrict__ bias,
                                                                     const float* __restrict__ window, const T* __restrict__ dy,
                                                                     T* __restrict__ dx, int64_t dxbs, int64_t dxrs,
                                                                     float* __restrict__ dwindow, float* __restrict__ part, int L,
                                                                     int C, int run, int cx, int nruns) {
  using P = Pairs<T, VEC>;
  using Raw = typename P::Raw;
  constexpr int BYTES = VEC * (int)sizeof(T);
  constexpr int NSTG = BYTES >= 16 ? 3 : 4;          // two rings: 48 KB of static shared memory at most
  __shared__ Raw ringx[NSTG][CS_ROWS][CS_THREADS];
  __shared__ Raw ringg[NSTG][CS_ROWS][CS_THREADS];
  const int tid = threadIdx.x;
  const int c0 = (blockIdx.y * cx + (tid & (cx - 1))) * VEC;
  const int b = blockIdx.z;
  const int ridx = blockIdx.x * (CS_THREADS / cx) + tid / cx;
  const int t0 = ridx * run;
  if (t0 >= L) return;
  const int ntok = min(run, L - t0);
  const int nrows = ntok + 2 * (W - 1);
  const int nst = (nrows + CS_ROWS - 1) / CS_ROWS;
  const T* xb = x + b * xbs + c0;
  const T* gb = dy + (int64_t)b * L * C + c0;
  auto issue = [&](int s) {
    if (s < nst) {
#pragma unroll
      for (int r = 0; r < CS_ROWS; ++r) {
        const int i = s * CS_ROWS + r, t = t0 - (W - 1) + i;
        const int st = s % NSTG;
        if (i < nrows && t < L) {
          if (t >= 0) cs_copy<BYTES>(&ringx[st][r][tid], xb + (int64_t)t * xrs);
          else ringx[st][r][tid] = window_row<T, VEC, W>(window, b, t, c0, C);
          if (i >= W - 1) cs_copy<BYTES>(&ringg[st][r][tid], gb + (int64_t)t * C);
        }
      }
    }
    cs_commit();
  };
  float2 w2[W][VEC / 2], b2[VEC / 2], dw2[W][VEC / 2], db2[VEC / 2];
#pragma unroll
  for (int s = 0; s < NSTG - 1; ++s) issue(s);
  load_taps2<VEC, W>(w2, b2, weight, bias, c0);
  P xr[W];                                              // xr[j] = input row of token t - (W-1) + j
  float2 dz[W][VEC / 2];                                // dz[k] = dz at token t - k
#pragma unroll
  for (int j = 0; j < W; ++j)
#pragma unroll
    for (int i = 0; i < VEC / 2; ++i) {
      xr[j].p[i] = make_float2(0.f, 0.f);
      dz[j][i] = make_float2(0.f, 0.f);
      dw2[j][i] = make_float2(0.f, 0.f);
    }
#pragma unroll
  for (int i = 0; i < VEC / 2; ++i) db2[i] = make_float2(0.f, 0.f);
  T* dxb = dx + b * dxbs + (int64_t)t0 * dxrs + c0;
  // one row of the walk; FULL: an owned token past both halos (x, dy present; dw / db taken; a dx row leaves): no tests
  auto row = [&](int s, int r, auto full) {
    constexpr bool FULL = decltype(full)::value;
    const int i = s * CS_ROWS + r;
    if (FULL || i < nrows) {
      const int t = t0 - (W - 1) + i;
      const int st = s % NSTG;
#pragma unroll
      for (int k = W - 1; k > 0; --k)
#pragma unroll
        for (int e = 0; e < VEC / 2; ++e) dz[k][e] = dz[k - 1][e];
      if (FULL || t < L) {
#pragma unroll
        for (int j = 0; j < W - 1; ++j) xr[j] = xr[j + 1];
        xr[W - 1].from_raw(ringx[st][r][tid]);
      }
      if (FULL || (t < L && i >= W - 1)) {
        P g;
        g.from_raw(ringg[st][r][tid]);
        const bool own = FULL || i < ntok + W - 1;
#pragma unroll
        for (int e = 0; e < VEC / 2; ++e) {
          float2 pre = b2[e];
#pragma unroll
          for (int j = 0; j < W; ++j) pre = fma2(w2[j][e], xr[j].p[e], pre);
          const float2 d = SILU ? mul2(g.p[e], silu_grad2<T>(pre)) : g.p[e];
          dz[0][e] = d;
          if (own) {
            db2[e] = add2(db2[e], d);
#pragma unroll
            for (int j = 0; j < W; ++j) dw2[j][e] = fma2(d, xr[j].p[e], dw2[j][e]);
          }
        }
      } else {
#pragma unroll
        for (int e = 0; e < VEC / 2; ++e) dz[0][e] = make_float2(0.f, 0.f);
      }
      if (FULL || i >= 2 * (W - 1)) {                   // dx of token t - (W-1) = sum_j w[j] dz(t - j)
        P o;
#pragma unroll
        for (int e = 0; e < VEC / 2; ++e) {
          float2 acc = mul2(w2[0][e], dz[0][e]);
#pragma unroll
          for (int j = 1; j < W; ++j) acc = fma2(w2[j][e], dz[j][e], acc);
          o.p[e] = acc;
        }
        *reinterpret_cast<Raw*>(dxb + (int64_t)(i - 2 * (W - 1)) * dxrs) = o.to_raw();
      } else if (!FULL && dwindow != nullptr && t0 == 0 && i >= W - 1) {
        // the first run also owns the gradient of the carried window: its slot W + tp is the input of token tp < 0
        const int tp = i - 2 * (W - 1);
#pragma unroll
        for (int e = 0; e < VEC / 2; ++e) {
          float2 acc = mul2(w2[0][e], dz[0][e]);
#pragma unroll
          for (int j = 1; j < W; ++j) acc = fma2(w2[j][e], dz[j][e], acc);
          dwindow[((int64_t)b * C + c0 + 2 * e) * W + (W + tp)] = acc.x;
          dwindow[((int64_t)b * C + c0 + 2 * e + 1) * W + (W + tp)] = acc.y;
        }
      }
    }
  };
  for (int s = 0; s < nst; ++s) {
    issue(s + NSTG - 1);
    cs_wait<NSTG - 1>();
    if (s * CS_ROWS >= 2 * (W - 1) && s * CS_ROWS + CS_ROWS <= ntok + W - 1) {
#pragma unroll
      for (int r = 0; r < CS_ROWS; ++r) row(s, r, std::true_type{});
    } else {
#pragma unroll
      for (int r = 0; r < CS_ROWS; ++r) row(s, r, std::false_type{});
    }
  }
  if (part != nullptr) {
    float* p = part + ((int64_t)(b * nruns + ridx) * C + c0) * (W + 1);
#pragma unroll
    for (int e = 0; e < VEC / 2; ++e) {
#pragma unroll
      for (int j = 0; j < W; ++j) {
        p[(2 * e) * (W + 1) + j] = dw2[j][e].x;
        p[(2 * e + 1) * (W + 1) + j] = dw2[j][e].y;
      }
      p[(2 * e) * (W + 1) + W] = db2[e].x;
      p[(2 * e + 1) * (W + 1) + W] = db2[e].y;
    }
  }
}

// Width of a CTA in channel vectors (0: the streaming kernels do not serve this channel count) and the token run of a
// thread: the longest of 256..32 that still leaves a few CTAs per SM slot (shorter runs only cost halo rows).
static inline int stream_cx(int C, int VEC) {
  if (C % VEC) return 0;
  const int cv = C / VEC;
  return cv % 128 == 0 ? 128 : (cv % 64 == 0 ? 64 : (cv % 32 == 0 ? 32 : 0));
}
static inline int stream_run(int B, int L, int cv, int cx) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int ty = CS_THREADS / cx;
  for (int run = 256; run > 32; run >>= 1) {
    const int64_t nr = (L + run - 1) / run;
    const int64_t ctas = (int64_t)B * ((nr + ty - 1) / ty) * (cv / cx);
    if (ctas >= (int64_t)sms * 12) return run;
  }
  return 32;
}

// out[c, k] = sum over partial slots in a fixed order (k < W -> dweight[c,k], k == W -> dbias[c]): a CTA owns 32
// columns; warp g sums the slots congruent to g modulo 8, then the 8 partial sums are added in order.
__global__ void __launch_bounds__(256) conv_reduce_kernel(const float* __restrict__ part, float* __restrict__ dweight,
                                                          float* __restrict__ dbias, int nslots, int C, int W) {
  __shared__ float red[8][33];
  const int lane = threadIdx.x & 31, grp = threadIdx.x >> 5;
  const int idx = blockIdx.x * 32 + lane, n = C * (W + 1);
  float acc = 0.f;
  if (idx < n) {
#pragma unroll 4
    for (int s = grp; s < nslots; s += 8) acc += part[(int64_t)s * n + idx];
  }
  red[grp][lane] = acc;
  __syncthreads();
  if (grp == 0 && idx < n) {
    float v = red[0][lane];
#pragma unroll
    for (int g = 1; g < 8; ++g) v += red[g][lane];
    const int c = idx / (W + 1), k = idx % (W + 1);
    if (k < W) dweight[c * W + k] = v;
    else if (dbias) dbias[c] = v;
  }
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
  if constexpr (VEC == 4) {   // the streaming kernels are built for 4 channels per thread (8 bytes bf16, 16 bytes fp32)
    if (const int cx = stream_cx(C, VEC)) {
      const int cv = C / VEC, run = stream_run(B, L, cv, cx), ty = CS_THREADS / cx;
      dim3 tg(((L + run - 1) / run + ty - 1) / ty, cv / cx, B);
      if (silu) conv_fwd_stream_kernel<T, VEC, W, true><<<tg, CS_THREADS, 0, st>>>(x, xbs, xrs, w, b, win, y, L, C, run, cx);
      else conv_fwd_stream_kernel<T, VEC, W, false><<<tg, CS_THREADS, 0, st>>>(x, xbs, xrs, w, b, win, y, L, C, run, cx);
      ORBIT_CHECK_LAUNCH("conv_fwd_stream_kernel");
      return OK;
    }
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
  if constexpr (VEC == 4) {
    const int cx = stream_cx(C, VEC);
    if (cx) {
      const int cv = C / VEC, run = stream_run(B, L, cv, cx), ty = CS_THREADS / cx, nruns = (L + run - 1) / run;
      *nslots = B * nruns;
      dim3 tg((nruns + ty - 1) / ty, cv / cx, B);
      if (silu) conv_bwd_stream_kernel<T, VEC, W, true><<<tg, CS_THREADS, 0, st>>>(x, xbs, xrs, w, b, win, dy, dx, dxbs, dxrs, dwin, part, L, C, run, cx, nruns);
      else conv_bwd_stream_kernel<T, VEC, W, false><<<tg, CS_THREADS, 0, st>>>(x, xbs, xrs, w, b, win, dy, dx, dxbs, dxrs, dwin, part, L, C, run, cx, nruns);
      ORBIT_CHECK_LAUNCH("conv_bwd_stream_kernel");
      return OK;
    }
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
      if (stream_cx(C, 4)) {   // streaming path: 8-byte channel vectors (measured faster than 16-byte ones: more warps resident)
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
        if (stream_cx(C, 4)) {   // streaming path: 8-byte channel vectors
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
    conv_reduce_kernel<<<(n + 31) / 32, 256, 0, st>>>(part, dweight, dbias, nslots, C, W);
    ORBIT_CHECK_LAUNCH("conv_reduce_kernel");
  }
  return OK;
}

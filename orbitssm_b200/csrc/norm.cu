// Output gate + RMSNorm, forward and backward:   out = rms_norm(y * silu(z)) * w
//
// Replaces the reference's fused gated norm (src/orbit_ssm/kernels/gated_norm.py:30-128, router
// src/orbit_ssm/layers/norms.py:133-168) and the gate epilogue it applies after the scan
// (src/orbit_ssm/ssm/ssd_mimo_torch.py:619-622).  Either half is optional: z == NULL -> plain RMSNorm,
// w == NULL -> gate only.  One CTA per row keeps the row in registers: a single pass over HBM.
// HBM-bound: forward 3*M*D*es bytes (y, z in; out), backward 5*M*D*es (y, z, dout in; dy, dz out).
#include "common.cuh"
#include "../../include/orbit_b200.h"
#include <mutex>

namespace orbit {

constexpr int NORM_THREADS = 256;
constexpr int NORM_MAXV = 4;   // 16-byte vectors per thread kept in registers


// Sums of ROWS values over the CTA with ONE barrier: warp sums go to red[r][warp], then every thread adds the 8 warp sums
// of each value in order.  `red` must not be rewritten before every thread has read it: callers alternate two buffers.
template <int ROWS>
__device__ __forceinline__ void block_sum_rows(float (&v)[ROWS], float (*red)[NORM_THREADS / 32]) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    v[r] = warp_sum(v[r]);
    if (lane == 0) red[r][wid] = v[r];
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    float t = red[r][0];
#pragma unroll
    for (int w = 1; w < NORM_THREADS / 32; ++w) t += red[r][w];
    v[r] = t;
  }
}

// Forward: a CTA owns ROWS consecutive rows (narrow rows are grouped so that a thread has several 16-byte loads in
// flight and the one barrier serves all of them); every load is issued before the first use.
template <typename T, int NV, int ROWS, bool GATED>
__global__ void __launch_bounds__(NORM_THREADS) gate_norm_fwd_kernel(const T* __restrict__ y,
                                                                     const T* __restrict__ z, int64_t zrs,
                                                                     const float* __restrict__ w, T* __restrict__ out,
                                                                     float* __restrict__ rstd_out, int64_t M, int D, float eps) {
  constexpr int V = Vec16<T>::N;
  __shared__ float red[ROWS][NORM_THREADS / 32];
  const int64_t row0 = (int64_t)blockIdx.x * ROWS;
  Vec16<T> ra[ROWS][NV], rb[ROWS][NV];
#pragma unroll
  for (int r = 0; r < ROWS; ++r)
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int c = (k * NORM_THREADS + threadIdx.x) * V;
      if (c < D && row0 + r < M) {
        ra[r][k].load(y + (row0 + r) * D + c);
        if (GATED) rb[r][k].load(z + (row0 + r) * zrs + c);
      }
    }
  float g[ROWS][NV][V], ss[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    ss[r] = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int c = (k * NORM_THREADS + threadIdx.x) * V;
      if (c < D && row0 + r < M) {
#pragma unroll
        for (int i = 0; i < V; ++i) {
          g[r][k][i] = GATED ? ra[r][k].get(i) * silu_t<T>(rb[r][k].get(i)) : ra[r][k].get(i);
          ss[r] = fmaf(g[r][k][i], g[r][k][i], ss[r]);
        }
      }
    }
  }
  float rstd[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) rstd[r] = 1.f;
  if (w != nullptr) {
    block_sum_rows<ROWS>(ss, red);
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      rstd[r] = rsqrtf(ss[r] / (float)D + eps);
      if (threadIdx.x == 0 && rstd_out && row0 + r < M) rstd_out[row0 + r] = rstd[r];
    }
  }
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int c = (k * NORM_THREADS + threadIdx.x) * V;
    if (c < D) {
      float wv[V];
#pragma unroll
      for (int i = 0; i < V; ++i) wv[i] = w ? w[c + i] : 1.f;
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        if (row0 + r < M) {
          Vec16<T> o;
#pragma unroll
          for (int i = 0; i < V; ++i) o.set(i, w ? g[r][k][i] * rstd[r] * wv[i] : g[r][k][i]);
          o.store(out + (row0 + r) * D + c);
        }
      }
    }
  }
}

// Backward: each CTA walks groups of ROWS rows (group blockIdx.x, blockIdx.x + gridDim.x, ...); dw partial sums stay in
// registers and go to `part` [gridDim.x, D] (fixed-order second stage below -> deterministic).
//   xh = g*rstd, u = dout*w, m = mean(xh*u), dg = rstd*(u - xh*m), dy = dg*silu(z), dz = dg*y*silu'(z)
template <typename T, int NV, int ROWS, bool GATED>
__global__ void __launch_bounds__(NORM_THREADS, (GATED && NV == 4) ? 1 : 2) gate_norm_bwd_kernel(
    const T* __restrict__ y, const T* __restrict__ z, int64_t zrs, const float* __restrict__ w,
    const float* __restrict__ rstd_in, const T* __restrict__ dout, T* __restrict__ dy, T* __restrict__ dz,
    int64_t dzrs, float* __restrict__ part, int64_t M, int D) {
  constexpr int V = Vec16<T>::N;
  __shared__ float red[2][ROWS][NORM_THREADS / 32];
  float dwacc[NV][V];
#pragma unroll
  for (int k = 0; k < NV; ++k)
#pragma unroll
    for (int i = 0; i < V; ++i) dwacc[k][i] = 0.f;
  // The row groups of a CTA are software-pipelined by one: the loads of the next group are issued before the block-wide sum
  // of the current one, so they are in flight across its barrier and the output pass.  (A deeper cp.async ring through shared
  // memory was measured slower: the kernel is not bound by load latency.)
  Vec16<T> ra[ROWS][NV], rd[ROWS][NV], rb[GATED ? ROWS : 1][NV];
  auto fetch = [&](int64_t row0) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int c = (k * NORM_THREADS + threadIdx.x) * V;
        if (c < D && row0 + r < M) {
          ra[r][k].load(y + (row0 + r) * D + c);
          rd[r][k].load(dout + (row0 + r) * D + c);
          if (GATED) rb[GATED ? r : 0][k].load(z + (row0 + r) * zrs + c);
        }
      }
  };
  const int64_t stride = (int64_t)gridDim.x * ROWS;
  if ((int64_t)blockIdx.x * ROWS < M) fetch((int64_t)blockIdx.x * ROWS);
  float wv[NV][V];                                    // the norm weights of this thread's columns, once per kernel
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int c = (k * NORM_THREADS + threadIdx.x) * V;
#pragma unroll
    for (int i = 0; i < V; ++i) wv[k][i] = (w != nullptr && c < D) ? w[c + i] : 1.f;
  }
  int par = 0;
  for (int64_t row0 = (int64_t)blockIdx.x * ROWS; row0 < M; row0 += stride, par ^= 1) {
    float yv[ROWS][NV][V], sz[GATED ? ROWS : 1][NV][V], gz[GATED ? ROWS : 1][NV][V], u[ROWS][NV][V];
    float rstd[ROWS], dot[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      rstd[r] = (w && row0 + r < M) ? rstd_in[row0 + r] : 1.f;
      dot[r] = 0.f;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int c = (k * NORM_THREADS + threadIdx.x) * V;
        if (c < D && row0 + r < M) {
#pragma unroll
          for (int i = 0; i < V; ++i) {
            float s1 = 1.f;
            if (GATED) {
              const float zz = rb[GATED ? r : 0][k].get(i);
              s1 = silu_t<T>(zz);
              sz[GATED ? r : 0][k][i] = s1;
              gz[GATED ? r : 0][k][i] = silu_grad_t<T>(zz);
            }
            yv[r][k][i] = ra[r][k].get(i);
            const float dd = rd[r][k].get(i);
            if (w != nullptr) {
              const float xh = yv[r][k][i] * s1 * rstd[r];
              u[r][k][i] = dd * wv[k][i];
              dot[r] = fmaf(xh, u[r][k][i], dot[r]);
              dwacc[k][i] = fmaf(dd, xh, dwacc[k][i]);
            } else {
              u[r][k][i] = dd;
            }
          }
        }
      }
    }
    if (row0 + stride < M) fetch(row0 + stride);
    if (w != nullptr) block_sum_rows<ROWS>(dot, red[par]);
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const float m = dot[r] / (float)D;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int c = (k * NORM_THREADS + threadIdx.x) * V;
        if (c < D && row0 + r < M) {
          Vec16<T> oy, oz;
#pragma unroll
          for (int i = 0; i < V; ++i) {
            const float s1 = GATED ? sz[GATED ? r : 0][k][i] : 1.f;
            float dg = u[r][k][i];
            if (w != nullptr) {
              const float xh = yv[r][k][i] * s1 * rstd[r];
              dg = rstd[r] * (u[r][k][i] - xh * m);
            }
            oy.set(i, dg * s1);
            if (GATED) oz.set(i, dg * yv[r][k][i] * gz[GATED ? r : 0][k][i]);
          }
          oy.store(dy + (row0 + r) * D + c);
          if (GATED) oz.store(dz + (row0 + r) * dzrs + c);
        }
      }
    }
  }
  if (part != nullptr) {
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      int c = (k * NORM_THREADS + threadIdx.x) * V;
      if (c < D) {
#pragma unroll
        for (int i = 0; i < V; ++i) part[(int64_t)blockIdx.x * D + c + i] = dwacc[k][i];
      }
    }
  }
}

// Scalar variants for widths or strides that are not multiples of a 16-byte vector (small test geometries).
template <typename T>
__global__ void __launch_bounds__(NORM_THREADS) gate_norm_fwd_scalar_kernel(const T* __restrict__ y, const T* __restrict__ z,
                                                                            int64_t zrs, const float* __restrict__ w,
                                                                            T* __restrict__ out, float* __restrict__ rstd_out,
                                                                            int D, float eps) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  float ss = 0.f;
  for (int c = threadIdx.x; c < D; c += NORM_THREADS) {
    float g = ldf(y + row * D + c);
    if (z) g *= silu_t<T>(ldf(z + row * zrs + c));
    ss = fmaf(g, g, ss);
  }
  float rstd = 1.f;
  if (w != nullptr) {
    ss = block_sum(ss, red);
    rstd = rsqrtf(ss / (float)D + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
  }
  for (int c = threadIdx.x; c < D; c += NORM_THREADS) {
    float g = ldf(y + row * D + c);
    if (z) g *= silu_t<T>(ldf(z + row * zrs + c));
    stf(out + row * D + c, w ? g * rstd * w[c] : g);
  }
}

template <typename T>
__global__ void __launch_bounds__(NORM_THREADS) gate_norm_bwd_scalar_kernel(
    const T* __restrict__ y, const T* __restrict__ z, int64_t zrs, const float* __restrict__ w,
    const float* __restrict__ rstd_in, const T* __restrict__ dout, T* __restrict__ dy, T* __restrict__ dz, int64_t dzrs,
    float* __restrict__ part, int64_t M, int D) {
  __shared__ float red[32];
  bool first = true;
  for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
    const float rstd = w ? rstd_in[row] : 1.f;
    float dot = 0.f;
    if (w != nullptr) {
      for (int c = threadIdx.x; c < D; c += NORM_THREADS) {
        float sz = z ? silu_t<T>(ldf(z + row * zrs + c)) : 1.f;
        float xh = ldf(y + row * D + c) * sz * rstd;
        float dd = ldf(dout + row * D + c);
        dot = fmaf(xh, dd * w[c], dot);
        float* p = part + (int64_t)blockIdx.x * D + c;
        *p = (first ? 0.f : *p) + dd * xh;
      }
    }
    float m = w ? block_sum(dot, red) / (float)D : 0.f;
    for (int c = threadIdx.x; c < D; c += NORM_THREADS) {
      float zz = z ? ldf(z + row * zrs + c) : 0.f;
      float sz = z ? silu_t<T>(zz) : 1.f;
      float yv = ldf(y + row * D + c);
      float dg = ldf(dout + row * D + c);
      if (w != nullptr) {
        float xh = yv * sz * rstd;
        dg = rstd * (dg * w[c] - xh * m);
      }
      stf(dy + row * D + c, dg * sz);
      if (z) stf(dz + row * dzrs + c, dg * yv * silu_grad_t<T>(zz));
    }
    first = false;
  }
}

// out[c] = sum over partial slots in a fixed order: a CTA owns 32 columns, warp g sums the slots congruent to g modulo 8,
// then the 8 partial sums are added in order (deterministic; 8 x the loads in flight of a single walk).
__global__ void __launch_bounds__(256) colsum_kernel(const float* __restrict__ part, float* __restrict__ out, int nslots, int D) {
  __shared__ float red[8][33];
  const int lane = threadIdx.x & 31, grp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float acc = 0.f;
  if (c < D) {
#pragma unroll 4
    for (int s = grp; s < nslots; s += 8) acc += part[(int64_t)s * D + c];
  }
  red[grp][lane] = acc;
  __syncthreads();
  if (grp == 0 && c < D) {
    float v = red[0][lane];
#pragma unroll
    for (int g = 1; g < 8; ++g) v += red[g][lane];
    out[c] = v;
  }
}

static int norm_bwd_slots(int64_t M) {
  int64_t g = 148 * 4;
  return (int)(M < g ? (M > 0 ? M : 1) : g);
}

template <typename T>
static int norm_nv(int D) {
  constexpr int V = Vec16<T>::N;
  int per = NORM_THREADS * V;
  return (D + per - 1) / per;
}

}  // namespace orbit

using namespace orbit;

extern "C" int64_t orbit_gate_norm_bwd_workspace_bytes(int64_t M, int D) {
  return (int64_t)norm_bwd_slots(M) * D * (int64_t)sizeof(float);
}

template <typename T>
static int gate_norm_fwd_t(const void* y, const void* z, int64_t zrs, const float* w, void* out, float* rstd,
                           int64_t M, int D, float eps, cudaStream_t st) {
  constexpr int V = Vec16<T>::N;
  dim3 grid((unsigned)M);
  int nv = norm_nv<T>(D);
  const bool vec = D % V == 0 && (z == nullptr || zrs % V == 0) && aligned16(y) && aligned16(out) &&
                   (z == nullptr || aligned16(z)) && nv <= NORM_MAXV;
  if (!vec) {
    gate_norm_fwd_scalar_kernel<T><<<grid, NORM_THREADS, 0, st>>>((const T*)y, (const T*)z, zrs, w, (T*)out, rstd, D, eps);
    ORBIT_CHECK_LAUNCH("gate_norm_fwd_scalar_kernel");
    return OK;
  }
  // a gate doubles the bytes per row; ungated narrow rows (the backbone norms) are grouped 4 or 2 to a CTA
#define L_(NV, ROWS, G) gate_norm_fwd_kernel<T, NV, ROWS, G><<<(unsigned)((M + ROWS - 1) / ROWS), NORM_THREADS, 0, st>>>((const T*)y, (const T*)z, zrs, w, (T*)out, rstd, M, D, eps)
  if (z != nullptr) { if (nv <= 1) L_(1, 4, true); else if (nv == 2) L_(2, 2, true); else L_(4, 1, true); }
  else { if (nv <= 1) L_(1, 4, false); else if (nv == 2) L_(2, 2, false); else L_(4, 1, false); }
#undef L_
  ORBIT_CHECK_LAUNCH("gate_norm_fwd_kernel");
  return OK;
}

extern "C" int orbit_gate_norm_fwd(const void* y, const void* z, int64_t z_row_stride, const float* w, void* out,
                                   float* rstd, int64_t M, int D, float eps, int dtype, void* stream) {
  ORBIT_REQUIRE(y && out, ERR_BAD_ARG, "orbit_gate_norm_fwd: null y/out");
  ORBIT_REQUIRE(M >= 0 && D > 0, ERR_BAD_ARG, "orbit_gate_norm_fwd: bad sizes M=%lld D=%d", (long long)M, D);
  ORBIT_REQUIRE(w == nullptr || rstd != nullptr, ERR_BAD_ARG, "orbit_gate_norm_fwd: rstd is required with a norm");
  if (M == 0) return OK;
  if (dtype == BF16) return gate_norm_fwd_t<__nv_bfloat16>(y, z, z_row_stride, w, out, rstd, M, D, eps, (cudaStream_t)stream);
  if (dtype == F32) return gate_norm_fwd_t<float>(y, z, z_row_stride, w, out, rstd, M, D, eps, (cudaStream_t)stream);
  return fail(ERR_BAD_ARG, "orbit_gate_norm_fwd: unknown dtype code %d", dtype);
}

template <typename T>
static int gate_norm_bwd_t(const void* y, const void* z, int64_t zrs, const float* w, const float* rstd,
                           const void* dout, void* dy, void* dz, int64_t dzrs, float* dw, float* part, int64_t M,
                           int D, cudaStream_t st) {
  constexpr int V = Vec16<T>::N;
  int nv = norm_nv<T>(D);
  int slots = norm_bwd_slots(M);
  dim3 grid(slots);
  const bool vec = D % V == 0 && (z == nullptr || (zrs % V == 0 && dzrs % V == 0)) && aligned16(y) && aligned16(dout) &&
                   aligned16(dy) && (z == nullptr || (aligned16(z) && aligned16(dz))) && nv <= NORM_MAXV;
  if (!vec) {
    gate_norm_bwd_scalar_kernel<T><<<grid, NORM_THREADS, 0, st>>>((const T*)y, (const T*)z, zrs, w, rstd, (const T*)dout,
                                                                  (T*)dy, (T*)dz, dzrs, part, M, D);
    ORBIT_CHECK_LAUNCH("gate_norm_bwd_scalar_kernel");
    if (dw != nullptr) {
      colsum_kernel<<<(D + 31) / 32, 256, 0, st>>>(part, dw, slots, D);
      ORBIT_CHECK_LAUNCH("colsum_kernel");
    }
    return OK;
  }
#define L_(NV, ROWS, G) gate_norm_bwd_kernel<T, NV, ROWS, G><<<grid, NORM_THREADS, 0, st>>>((const T*)y, (const T*)z, zrs, w, rstd, (const T*)dout, (T*)dy, (T*)dz, dzrs, part, M, D)
  if (z != nullptr) { if (nv <= 1) L_(1, 2, true); else if (nv == 2) L_(2, 1, true); else L_(4, 1, true); }
  else { if (nv <= 1) L_(1, 4, false); else if (nv == 2) L_(2, 2, false); else L_(4, 1, false); }
#undef L_
  ORBIT_CHECK_LAUNCH("gate_norm_bwd_kernel");
  if (dw != nullptr) {
    colsum_kernel<<<(D + 31) / 32, 256, 0, st>>>(part, dw, slots, D);
    ORBIT_CHECK_LAUNCH("colsum_kernel");
  }
  return OK;
}

extern "C" int orbit_gate_norm_bwd(const void* y, const void* z, int64_t z_row_stride, const float* w,
                                   const float* rstd, const void* dout, void* dy, void* dz, int64_t dz_row_stride,
                                   float* dw, void* workspace, int64_t workspace_bytes, int64_t M, int D, int dtype,
                                   void* stream) {
  ORBIT_REQUIRE(y && dout && dy, ERR_BAD_ARG, "orbit_gate_norm_bwd: null y/dout/dy");
  ORBIT_REQUIRE(z == nullptr || dz != nullptr, ERR_BAD_ARG, "orbit_gate_norm_bwd: dz is required with a gate");
  ORBIT_REQUIRE(w == nullptr || (rstd != nullptr && dw != nullptr), ERR_BAD_ARG,
                "orbit_gate_norm_bwd: rstd and dw are required with a norm");
  ORBIT_REQUIRE(M >= 0 && D > 0, ERR_BAD_ARG, "orbit_gate_norm_bwd: bad sizes M=%lld D=%d", (long long)M, D);
  cudaStream_t st = (cudaStream_t)stream;
  if (M == 0) {
    if (dw) ORBIT_CHECK_CUDA(cudaMemsetAsync(dw, 0, sizeof(float) * D, st));
    return OK;
  }
  float* part = nullptr;
  if (w != nullptr) {
    ORBIT_REQUIRE(workspace && workspace_bytes >= orbit_gate_norm_bwd_workspace_bytes(M, D), ERR_WORKSPACE,
                  "orbit_gate_norm_bwd: workspace of %lld bytes needed",
                  (long long)orbit_gate_norm_bwd_workspace_bytes(M, D));
    part = (float*)workspace;
  }
  if (dtype == BF16)
    return gate_norm_bwd_t<__nv_bfloat16>(y, z, z_row_stride, w, rstd, dout, dy, dz, dz_row_stride, dw, part, M, D, st);
  if (dtype == F32)
    return gate_norm_bwd_t<float>(y, z, z_row_stride, w, rstd, dout, dy, dz, dz_row_stride, dw, part, M, D, st);
  return fail(ERR_BAD_ARG, "orbit_gate_norm_bwd: unknown dtype code %d", dtype);
}


// ---- gate + RMSNorm backward without any allocation ---------------------------------------------------------------
// Same arithmetic as orbit_gate_norm_bwd; the partial-sum buffer of the weight gradient lives in this file-scope device
// array instead of a caller workspace.  Every GPU that loads the library holds the array (9.25 MiB) until exit.
namespace orbit {
constexpr int64_t NORM_NOALLOC_FLOATS = 592LL * 4096;   // slots(M) * D must fit: e.g. any M with D <= 4096
static __device__ __align__(256) float g_norm_bwd_scratch[NORM_NOALLOC_FLOATS];

// In host code the array's name is only a handle; the device address comes from cudaGetSymbolAddress, asked once per
// device with that device current.
static float* g_norm_bwd_scratch_ptr[64] = {nullptr};
static std::mutex g_norm_bwd_scratch_mu;

static int norm_noalloc_scratch(float** out) {
  int dev = -1;
  ORBIT_CHECK_CUDA(cudaGetDevice(&dev));
  ORBIT_REQUIRE(dev >= 0 && dev < 64, ERR_UNSUPPORTED, "orbit_gate_norm_bwd_noalloc: device index %d outside 0..63", dev);
  std::lock_guard<std::mutex> lock(g_norm_bwd_scratch_mu);
  if (g_norm_bwd_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    ORBIT_CHECK_CUDA(cudaGetSymbolAddress(&p, g_norm_bwd_scratch));
    ORBIT_REQUIRE(p != nullptr, ERR_CUDA, "orbit_gate_norm_bwd_noalloc: cudaGetSymbolAddress returned a null address");
    g_norm_bwd_scratch_ptr[dev] = (float*)p;
  }
  *out = g_norm_bwd_scratch_ptr[dev];
  return OK;
}
}  // namespace orbit

extern "C" int orbit_gate_norm_bwd_noalloc(const void* y, const void* z, int64_t z_row_stride, const float* w,
                                           const float* rstd, const void* dout, void* dy, void* dz,
                                           int64_t dz_row_stride, float* dw, int64_t M, int D, int dtype, void* stream) {
  ORBIT_REQUIRE(y && dout && dy, ERR_BAD_ARG, "orbit_gate_norm_bwd_noalloc: null y/dout/dy");
  ORBIT_REQUIRE(z == nullptr || dz != nullptr, ERR_BAD_ARG, "orbit_gate_norm_bwd_noalloc: dz is required with a gate");
  ORBIT_REQUIRE(w == nullptr || (rstd != nullptr && dw != nullptr), ERR_BAD_ARG,
                "orbit_gate_norm_bwd_noalloc: rstd and dw are required with a norm");
  ORBIT_REQUIRE(M >= 0 && D > 0, ERR_BAD_ARG, "orbit_gate_norm_bwd_noalloc: bad sizes M=%lld D=%d", (long long)M, D);
  cudaStream_t st = (cudaStream_t)stream;
  if (M == 0) {
    if (dw) ORBIT_CHECK_CUDA(cudaMemsetAsync(dw, 0, sizeof(float) * D, st));
    return OK;
  }
  float* part = nullptr;
  if (w != nullptr) {
    // Only the weight gradient needs scratch: a gate-only call (w == NULL) of any size is served.
    const int64_t need = (int64_t)norm_bwd_slots(M) * D;
    ORBIT_REQUIRE(need <= NORM_NOALLOC_FLOATS, ERR_UNSUPPORTED,
                  "orbit_gate_norm_bwd_noalloc: min(M, 592) * D = %lld floats of scratch exceed the built-in %lld (M=%lld, D=%d); "
                  "use orbit_gate_norm_bwd with a caller workspace", (long long)need, (long long)NORM_NOALLOC_FLOATS,
                  (long long)M, D);
    // The built-in array is per device and its address is looked up for the CURRENT device: the buffers must live there
    // too, or the kernel would be handed another GPU's scratch.
    int dev = -1;
    ORBIT_CHECK_CUDA(cudaGetDevice(&dev));
    cudaPointerAttributes attr;
    ORBIT_CHECK_CUDA(cudaPointerGetAttributes(&attr, dy));
    ORBIT_REQUIRE(attr.type != cudaMemoryTypeDevice || attr.device == dev, ERR_BAD_ARG,
                  "orbit_gate_norm_bwd_noalloc: dy lives on device %d but the current device is %d; make the buffers' device "
                  "current before the call", attr.device, dev);
    int rc = norm_noalloc_scratch(&part);
    if (rc != OK) return rc;
    // nothing in the scratch has to start at zero: each CTA overwrites its whole row of partial sums before the
    // fixed-order column sum reads exactly the rows that were written
  }
  if (dtype == BF16)
    return gate_norm_bwd_t<__nv_bfloat16>(y, z, z_row_stride, w, rstd, dout, dy, dz, dz_row_stride, dw, part, M, D, st);
  if (dtype == F32)
    return gate_norm_bwd_t<float>(y, z, z_row_stride, w, rstd, dout, dy, dz, dz_row_stride, dw, part, M, D, st);
  return fail(ERR_BAD_ARG, "orbit_gate_norm_bwd_noalloc: unknown dtype code %d", dtype);
}

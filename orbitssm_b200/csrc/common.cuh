// Shared device/host helpers of the orbit_b200 C-ABI library (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>

namespace orbit {

// Status codes returned by every extern "C" entry point (0 = ok).  The text of the last failure on the
// calling thread is available from orbit_last_error().
enum Status : int {
  OK = 0,
  ERR_BAD_ARG = 1,        // null pointer, negative size, unknown dtype code
  ERR_UNSUPPORTED = 2,    // shape/alignment outside the kernel's envelope (named in the message)
  ERR_CUDA = 3,           // a CUDA runtime call failed (message carries cudaGetErrorString)
  ERR_WORKSPACE = 4,      // workspace too small
  ERR_DEVICE_TIMEOUT = 5  // a bounded device-side wait gave up (status word set by the kernel)
};

enum DType : int { F32 = 0, BF16 = 1 };

void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);

#define ORBIT_CHECK_CUDA(expr)                                                         \
  do {                                                                                 \
    cudaError_t _e = (expr);                                                           \
    if (_e != cudaSuccess)                                                             \
      return ::orbit::fail(::orbit::ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)

#define ORBIT_CHECK_LAUNCH(name)                                                        \
  do {                                                                                  \
    cudaError_t _e = cudaGetLastError();                                                \
    if (_e != cudaSuccess)                                                              \
      return ::orbit::fail(::orbit::ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(_e)); \
  } while (0)

#define ORBIT_REQUIRE(cond, code, ...)                      \
  do {                                                      \
    if (!(cond)) return ::orbit::fail(code, __VA_ARGS__);   \
  } while (0)

// ---- element access -------------------------------------------------------------------------------
__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

template <typename T> struct Vec16;   // 16-byte vector of T
template <> struct Vec16<float> {
  static constexpr int N = 4;
  float4 v;
  __device__ __forceinline__ void load(const float* p) { v = *reinterpret_cast<const float4*>(p); }
  __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = v; }
  __device__ __forceinline__ float get(int i) const { return reinterpret_cast<const float*>(&v)[i]; }
  __device__ __forceinline__ void set(int i, float x) { reinterpret_cast<float*>(&v)[i] = x; }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  uint4 v;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { v = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void store(__nv_bfloat16* p) const { *reinterpret_cast<uint4*>(p) = v; }
  __device__ __forceinline__ float get(int i) const {
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(&v)[i]);
  }
  __device__ __forceinline__ void set(int i, float x) {
    reinterpret_cast<__nv_bfloat16*>(&v)[i] = __float2bfloat16_rn(x);
  }
};

__device__ __forceinline__ float sigmoidf_(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }
__device__ __forceinline__ float tanh_approx_(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Activation arithmetic by IO dtype: fp32 activations keep ~2 ulp sigmoids; bfloat16 activations (eps 2^-8) take the
// single-MUFU tanh form (abs error ~2^-11), which keeps the HBM-bound kernels from becoming issue-bound.
template <typename T> struct Act {
  static __device__ __forceinline__ float sigmoid(float x) { return sigmoidf_(x); }
};
template <> struct Act<__nv_bfloat16> {
  static __device__ __forceinline__ float sigmoid(float x) { return fmaf(0.5f, tanh_approx_(0.5f * x), 0.5f); }
};
template <typename T> __device__ __forceinline__ float silu_t(float x) { return x * Act<T>::sigmoid(x); }
template <typename T> __device__ __forceinline__ float silu_grad_t(float x) {
  float s = Act<T>::sigmoid(x);
  return s * fmaf(x, 1.f - s, 1.f);
}
__device__ __forceinline__ float siluf_(float x) { return x * sigmoidf_(x); }
// d/dx silu(x) = s (1 + x (1 - s))
__device__ __forceinline__ float silu_gradf_(float x) {
  float s = sigmoidf_(x);
  return s * (1.f + x * (1.f - s));
}

// Packed fp32 pairs (one instruction for two lanes of arithmetic: the per-element passes of these kernels are bound by
// instruction issue, not by the FP32 pipes).
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmul.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}
__device__ __forceinline__ float2 f2(uint32_t a, uint32_t b) { return make_float2(__uint_as_float(a), __uint_as_float(b)); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void unpack_bf16(uint32_t w, float& lo, float& hi) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&w);
  lo = __low2float(v);
  hi = __high2float(v);
}

__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tadd.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Block-wide sum; `red` is shared scratch of >= 32 floats; every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[wid] = v;
  __syncthreads();
  float t = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
  if (wid == 0) {
    t = warp_sum(t);
    if (lane == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace orbit

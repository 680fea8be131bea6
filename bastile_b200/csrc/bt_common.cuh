// Shared host/device helpers of the bastile_b200 kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/bastile_b200.h"

namespace bt {

// ---------------------------------------------------------------- errors
void set_error(const char* fmt, ...);  // defined in c_api.cu (thread-local text)

#define BT_CHECK_ARG(cond, ...)      \
  do {                               \
    if (!(cond)) {                   \
      ::bt::set_error(__VA_ARGS__);  \
      return BT_ERR_ARG;             \
    }                                \
  } while (0)

#define BT_CHECK_LAUNCH(what)                                                \
  do {                                                                       \
    cudaError_t e__ = cudaGetLastError();                                    \
    if (e__ != cudaSuccess) {                                                \
      ::bt::set_error("%s: %s", (what), cudaGetErrorString(e__));            \
      return BT_ERR_LAUNCH;                                                  \
    }                                                                        \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int sm_count();  // cached per device (c_api.cu)

// ---------------------------------------------------------------- 16-byte vectors
__device__ __forceinline__ uint4 ld_global_v4(const void* p) {
  return *reinterpret_cast<const uint4*>(p);
}
// Streaming variants: data that is touched exactly once should not displace the
// weights / cos / sin rows that every CTA re-reads.
__device__ __forceinline__ uint4 ld_stream_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_global_v4(void* p, uint4 v) {
  *reinterpret_cast<uint4*>(p) = v;
}
// Cache-streaming forms (evict-first in L1 and L2) for large tensors that a kernel touches
// once while other data - GEMM operand tiles - should stay resident in L2.
__device__ __forceinline__ uint4 ld_once_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_once_v4(void* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

// unpack / pack one 16-byte vector to fp32 lanes
template <typename T>
struct Cvt;

template <>
struct Cvt<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ __forceinline__ static void unpack(uint4 v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ __forceinline__ static uint4 pack(const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  __device__ __forceinline__ static float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
  __device__ __forceinline__ static __nv_bfloat16 from_f(float x) { return __float2bfloat16_rn(x); }
};

template <>
struct Cvt<__half> {
  static constexpr int N = 8;
  __device__ __forceinline__ static void unpack(uint4 v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
      float2 t = __half22float2(h);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
  __device__ __forceinline__ static uint4 pack(const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  __device__ __forceinline__ static float to_f(__half x) { return __half2float(x); }
  __device__ __forceinline__ static __half from_f(float x) { return __float2half_rn(x); }
};

template <>
struct Cvt<float> {
  static constexpr int N = 4;
  __device__ __forceinline__ static void unpack(uint4 v, float (&f)[4]) {
    f[0] = __uint_as_float(v.x);
    f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z);
    f[3] = __uint_as_float(v.w);
  }
  __device__ __forceinline__ static uint4 pack(const float (&f)[4]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                      __float_as_uint(f[3]));
  }
  __device__ __forceinline__ static float to_f(float x) { return x; }
  __device__ __forceinline__ static float from_f(float x) { return x; }
};

// ---------------------------------------------------------------- packed fp32 pairs
// sm_100 issues fp32 add / mul / fma on PAIRS of values held in a 64-bit register
// (fma.rn.f32x2 and friends): same IEEE results per lane, half the issue slots.  The row
// kernels are bound by instruction issue (a few resident warps per scheduler), not by
// arithmetic throughput, so their inner loops work on pairs.
struct f32x2 {
  unsigned long long r;
};
__device__ __forceinline__ f32x2 pair(float lo, float hi) {
  f32x2 p;
  asm("mov.b64 %0, {%1, %2};" : "=l"(p.r) : "f"(lo), "f"(hi));
  return p;
}
__device__ __forceinline__ float lo_of(f32x2 p) {
  float lo, hi;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(p.r));
  return lo;
}
__device__ __forceinline__ float hi_of(f32x2 p) {
  float lo, hi;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(p.r));
  return hi;
}
__device__ __forceinline__ f32x2 neg2(f32x2 a) {  // flips both sign bits
  f32x2 d;
  d.r = a.r ^ 0x8000000080000000ull;
  return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d.r) : "l"(a.r), "l"(b.r));
  return d;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d.r) : "l"(a.r), "l"(b.r));
  return d;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d.r) : "l"(a.r), "l"(b.r), "l"(c.r));
  return d;
}
// A 16-byte vector as fp32 pairs (N / 2 of them) and back.
template <typename T>
__device__ __forceinline__ void unpack_pairs(uint4 v, f32x2 (&p)[Cvt<T>::N / 2]) {
  float f[Cvt<T>::N];
  Cvt<T>::unpack(v, f);
#pragma unroll
  for (int i = 0; i < Cvt<T>::N / 2; ++i) p[i] = pair(f[2 * i], f[2 * i + 1]);
}
template <typename T>
__device__ __forceinline__ uint4 pack_pairs(const f32x2 (&p)[Cvt<T>::N / 2]) {
  float f[Cvt<T>::N];
#pragma unroll
  for (int i = 0; i < Cvt<T>::N / 2; ++i) {
    f[2 * i] = lo_of(p[i]);
    f[2 * i + 1] = hi_of(p[i]);
  }
  return Cvt<T>::pack(f);
}

// Tells the compiler that a packed 16-byte vector "changed": values unpacked from it before
// this point cannot be kept alive in registers across it and are recomputed from the packed
// form instead.  Costs nothing at run time; keeps two-pass row kernels at ~1 register per
// two elements instead of three.
__device__ __forceinline__ void forget_unpacked(uint4& v) {
  asm volatile("" : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w));
}

// Sum over the G consecutive lanes (G a power of two <= 32) that hold one row.
template <int G>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = G / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Programmatic dependent launch: a kernel launched through launch_dependent() may be set up on
// the SMs (its CTAs scheduled, their prologues run) while the previous kernel of the stream is
// still draining; it must call grid_dependency_wait() before its first access to global memory,
// which blocks until the previous kernel has completed and its writes are visible.  Launched
// the ordinary way the wait is a no-op.
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
int dependent_launch_mode();  // 1 (default): kernels are launched as programmatic dependents (c_api.cu)

template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = dependent_launch_mode() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

#define BT_CHECK_LAUNCHED(err, what)                                         \
  do {                                                                       \
    const cudaError_t e__ = (err);                                           \
    if (e__ != cudaSuccess) {                                                \
      ::bt::set_error("%s: %s", (what), cudaGetErrorString(e__));            \
      return BT_ERR_LAUNCH;                                                  \
    }                                                                        \
  } while (0)

// CTAs of `kern` that one SM holds at once (at least 1), for kernels whose grid should be exactly
// one wave.  `smem` is the dynamic shared memory of the launch (an upper bound is fine when it is
// small next to the SM's).
template <typename K>
inline int resident_ctas(K kern, int threads, size_t smem) {
  int n = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, threads, smem) != cudaSuccess || n < 1) {
    (void)cudaGetLastError();
    n = 1;
  }
  return n;
}

// RMSNorm backward scratch: K private copies of the N fp32 column sums (CTA b adds into
// copy b % K, which divides the same-address atomic traffic by K) followed by one arrival
// counter.  K * N stays within 16384 words.
__host__ __device__ inline int dw_copies(int64_t N) {
  const int64_t k = 16384 / (N > 0 ? N : 1);
  return k < 1 ? 1 : (k > 8 ? 8 : static_cast<int>(k));
}

// Adds 8 (or 4) consecutive fp32 values with 16-byte vector reductions.
__device__ __forceinline__ void red_add_v4(float* dst, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(a), "f"(b), "f"(c),
               "f"(d)
               : "memory");
}

// Last step of every RMSNorm backward kernel.  Each CTA has added its column sums into one
// of the dw_copies(N) private rows of the scratch; the CTA that draws the last ticket sums
// the copies into dw and leaves the scratch zeroed for the next call.  The reads are all
// issued before any of the zeroing stores so that they overlap instead of queueing up
// behind stores to the same array.
template <typename T>
__device__ __forceinline__ void dw_finalize(float* __restrict__ ws, T* __restrict__ dw, int N,
                                            unsigned int total_ctas, int tid, int nthreads) {
  __shared__ bool s_last;
  const int K = dw_copies(N);
  unsigned int* counter = reinterpret_cast<unsigned int*>(ws + static_cast<int64_t>(K) * N);
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned int ticket = atomicAdd(counter, 1u);
    s_last = (ticket == total_ctas - 1);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if ((N & 3) == 0) {
    const float4* ws4 = reinterpret_cast<const float4*>(ws);
    const int n4 = N >> 2;
#pragma unroll 2
    for (int c = tid; c < n4; c += nthreads) {
      float4 v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k)
        v[k] = k < K ? __ldcg(ws4 + static_cast<int64_t>(k) * n4 + c) : make_float4(0.f, 0.f, 0.f, 0.f);
      float o[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        o[0] += v[k].x;
        o[1] += v[k].y;
        o[2] += v[k].z;
        o[3] += v[k].w;
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) dw[c * 4 + e] = Cvt<T>::from_f(o[e]);
    }
  } else {
    for (int c = tid; c < N; c += nthreads) {
      float v = 0.f;
      for (int k = 0; k < K; ++k) v += __ldcg(ws + static_cast<int64_t>(k) * N + c);
      dw[c] = Cvt<T>::from_f(v);
    }
  }
  __syncthreads();
  const int64_t total = static_cast<int64_t>(K) * N;
  for (int64_t c = tid; c < total; c += nthreads) ws[c] = 0.f;
  if (tid == 0) *counter = 0u;
}

}  // namespace bt

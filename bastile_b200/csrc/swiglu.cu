// Stand-alone SwiGLU (silu(gate) * up) forward and backward for sm_100a.
// Pure streaming kernels: 16-byte accesses, several vectors in flight per
// thread, grid sized to a multiple of the SM count.
//
// Rounding points follow the operator being replaced: the forward rounds
// silu(gate) to the storage type and multiplies by `up` in that type (the
// product of two 16-bit floats is exact in fp32, so rounding the fp32 product
// once gives the same bits); the backward is fp32 throughout with an exact
// sigmoid and rounds dgate / dup once.
#include "bt_common.cuh"

namespace bt {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

__device__ __forceinline__ float sigmoid_fast(float g) {
  // exp via ex2.approx and an approximate reciprocal, denormals flushed.
  return __fdividef(1.0f, 1.0f + __expf(-g));
}
__device__ __forceinline__ float sigmoid_exact(float g) { return 1.0f / (1.0f + expf(-g)); }

template <typename T>
__global__ void __launch_bounds__(kThreads)
swiglu_fwd_vec(const T* __restrict__ gate, const T* __restrict__ up, T* __restrict__ out,
               int64_t rows, int vpr, int64_t ld_g, int64_t ld_u, int64_t ld_o) {
  constexpr int E = Cvt<T>::N;
  const int64_t total = rows * vpr;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t base = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; base < total;
       base += stride * kUnroll) {
    uint4 gv[kUnroll], uv[kUnroll];
    int64_t r[kUnroll];
    int c[kUnroll];
#pragma unroll
    for (int k = 0; k < kUnroll; ++k) {
      const int64_t idx = base + k * stride;
      r[k] = idx / vpr;
      c[k] = static_cast<int>(idx - r[k] * vpr) * E;
      if (idx < total) {
        gv[k] = ld_stream_v4(gate + r[k] * ld_g + c[k]);
        uv[k] = ld_stream_v4(up + r[k] * ld_u + c[k]);
      }
    }
#pragma unroll
    for (int k = 0; k < kUnroll; ++k) {
      if (base + k * stride < total) {
        float g[E], u[E], o[E];
        Cvt<T>::unpack(gv[k], g);
        Cvt<T>::unpack(uv[k], u);
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const float silu = Cvt<T>::to_f(Cvt<T>::from_f(g[e] * sigmoid_fast(g[e])));
          o[e] = silu * u[e];
        }
        st_global_v4(out + r[k] * ld_o + c[k], Cvt<T>::pack(o));
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
swiglu_bwd_vec(const T* __restrict__ dy, const T* __restrict__ gate, const T* __restrict__ up,
               T* __restrict__ dgate, T* __restrict__ dup, int64_t rows, int vpr, int64_t ld_dy,
               int64_t ld_g, int64_t ld_u, int64_t ld_dg, int64_t ld_du) {
  constexpr int E = Cvt<T>::N;
  constexpr int U = 2;
  const int64_t total = rows * vpr;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t base = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; base < total;
       base += stride * U) {
    uint4 yv[U], gv[U], uv[U];
    int64_t r[U];
    int c[U];
#pragma unroll
    for (int k = 0; k < U; ++k) {
      const int64_t idx = base + k * stride;
      r[k] = idx / vpr;
      c[k] = static_cast<int>(idx - r[k] * vpr) * E;
      if (idx < total) {
        yv[k] = ld_stream_v4(dy + r[k] * ld_dy + c[k]);
        gv[k] = ld_stream_v4(gate + r[k] * ld_g + c[k]);
        uv[k] = ld_stream_v4(up + r[k] * ld_u + c[k]);
      }
    }
#pragma unroll
    for (int k = 0; k < U; ++k) {
      if (base + k * stride < total) {
        float d[E], g[E], u[E], dg[E], du[E];
        Cvt<T>::unpack(yv[k], d);
        Cvt<T>::unpack(gv[k], g);
        Cvt<T>::unpack(uv[k], u);
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const float sg = sigmoid_exact(g[e]);
          dg[e] = d[e] * (sg * (1.0f + g[e] * (1.0f - sg))) * u[e];
          du[e] = d[e] * (g[e] * sg);
        }
        st_global_v4(dgate + r[k] * ld_dg + c[k], Cvt<T>::pack(dg));
        st_global_v4(dup + r[k] * ld_du + c[k], Cvt<T>::pack(du));
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
swiglu_fwd_scalar(const T* __restrict__ gate, const T* __restrict__ up, T* __restrict__ out,
                  int64_t rows, int64_t cols, int64_t ld_g, int64_t ld_u, int64_t ld_o) {
  const int64_t total = rows * cols;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * kThreads) {
    const int64_t r = idx / cols, c = idx - r * cols;
    const float g = Cvt<T>::to_f(gate[r * ld_g + c]);
    const float silu = Cvt<T>::to_f(Cvt<T>::from_f(g * sigmoid_fast(g)));
    out[r * ld_o + c] = Cvt<T>::from_f(silu * Cvt<T>::to_f(up[r * ld_u + c]));
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
swiglu_bwd_scalar(const T* __restrict__ dy, const T* __restrict__ gate, const T* __restrict__ up,
                  T* __restrict__ dgate, T* __restrict__ dup, int64_t rows, int64_t cols,
                  int64_t ld_dy, int64_t ld_g, int64_t ld_u, int64_t ld_dg, int64_t ld_du) {
  const int64_t total = rows * cols;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * kThreads) {
    const int64_t r = idx / cols, c = idx - r * cols;
    const float d = Cvt<T>::to_f(dy[r * ld_dy + c]);
    const float g = Cvt<T>::to_f(gate[r * ld_g + c]);
    const float u = Cvt<T>::to_f(up[r * ld_u + c]);
    const float sg = sigmoid_exact(g);
    dgate[r * ld_dg + c] = Cvt<T>::from_f(d * (sg * (1.0f + g * (1.0f - sg))) * u);
    dup[r * ld_du + c] = Cvt<T>::from_f(d * (g * sg));
  }
}

unsigned stream_grid(int64_t items_per_thread_total, int per_thread) {
  const int64_t blocks = ceil_div(items_per_thread_total, static_cast<int64_t>(kThreads) * per_thread);
  // whole waves: an SM holds 3 CTAs of these kernels at their register count, and a last wave that
  // is only partly full runs at a fraction of the bandwidth (8 per SM = 2.67 waves was 2 % slower)
  const int64_t cap = static_cast<int64_t>(sm_count()) * 12;
  return static_cast<unsigned>(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

template <typename T>
int fwd_t(const void* gate, const void* up, void* out, int64_t rows, int64_t cols, int64_t ld_g,
          int64_t ld_u, int64_t ld_o, cudaStream_t s) {
  constexpr int E = Cvt<T>::N;
  const bool vec_ok = cols % E == 0 && ld_g % E == 0 && ld_u % E == 0 && ld_o % E == 0 &&
                      aligned16(gate) && aligned16(up) && aligned16(out) && cols / E < (1ll << 31);
  if (vec_ok) {
    swiglu_fwd_vec<T><<<stream_grid(rows * (cols / E), kUnroll), kThreads, 0, s>>>(
        static_cast<const T*>(gate), static_cast<const T*>(up), static_cast<T*>(out), rows,
        static_cast<int>(cols / E), ld_g, ld_u, ld_o);
    BT_CHECK_LAUNCH("swiglu_fwd_vec");
  } else {
    swiglu_fwd_scalar<T><<<stream_grid(rows * cols, 1), kThreads, 0, s>>>(
        static_cast<const T*>(gate), static_cast<const T*>(up), static_cast<T*>(out), rows, cols,
        ld_g, ld_u, ld_o);
    BT_CHECK_LAUNCH("swiglu_fwd_scalar");
  }
  return BT_OK;
}

template <typename T>
int bwd_t(const void* dy, const void* gate, const void* up, void* dgate, void* dup, int64_t rows,
          int64_t cols, int64_t ld_dy, int64_t ld_g, int64_t ld_u, int64_t ld_dg, int64_t ld_du,
          cudaStream_t s) {
  constexpr int E = Cvt<T>::N;
  const bool vec_ok = cols % E == 0 && ld_dy % E == 0 && ld_g % E == 0 && ld_u % E == 0 &&
                      ld_dg % E == 0 && ld_du % E == 0 && aligned16(dy) && aligned16(gate) &&
                      aligned16(up) && aligned16(dgate) && aligned16(dup) &&
                      cols / E < (1ll << 31);
  if (vec_ok) {
    swiglu_bwd_vec<T><<<stream_grid(rows * (cols / E), 2), kThreads, 0, s>>>(
        static_cast<const T*>(dy), static_cast<const T*>(gate), static_cast<const T*>(up),
        static_cast<T*>(dgate), static_cast<T*>(dup), rows, static_cast<int>(cols / E), ld_dy,
        ld_g, ld_u, ld_dg, ld_du);
    BT_CHECK_LAUNCH("swiglu_bwd_vec");
  } else {
    swiglu_bwd_scalar<T><<<stream_grid(rows * cols, 1), kThreads, 0, s>>>(
        static_cast<const T*>(dy), static_cast<const T*>(gate), static_cast<const T*>(up),
        static_cast<T*>(dgate), static_cast<T*>(dup), rows, cols, ld_dy, ld_g, ld_u, ld_dg, ld_du);
    BT_CHECK_LAUNCH("swiglu_bwd_scalar");
  }
  return BT_OK;
}

}  // namespace
}  // namespace bt

extern "C" int bt_swiglu_fwd(const void* gate, const void* up, void* out, int64_t rows,
                             int64_t cols, int64_t ld_gate, int64_t ld_up, int64_t ld_out,
                             int dtype, void* stream) {
  using namespace bt;
  BT_CHECK_ARG(rows >= 0 && cols >= 0, "swiglu_fwd: negative size");
  if (rows == 0 || cols == 0) return BT_OK;
  BT_CHECK_ARG(gate && up && out, "swiglu_fwd: null pointer");
  BT_CHECK_ARG(ld_gate >= cols && ld_up >= cols && ld_out >= cols,
               "swiglu_fwd: row stride smaller than cols");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case BT_BF16: return fwd_t<__nv_bfloat16>(gate, up, out, rows, cols, ld_gate, ld_up, ld_out, s);
    case BT_FP16: return fwd_t<__half>(gate, up, out, rows, cols, ld_gate, ld_up, ld_out, s);
    case BT_FP32: return fwd_t<float>(gate, up, out, rows, cols, ld_gate, ld_up, ld_out, s);
  }
  set_error("swiglu_fwd: unknown dtype %d", dtype);
  return BT_ERR_ARG;
}

extern "C" int bt_swiglu_bwd(const void* dy, const void* gate, const void* up, void* dgate,
                             void* dup, int64_t rows, int64_t cols, int64_t ld_dy,
                             int64_t ld_gate, int64_t ld_up, int64_t ld_dgate, int64_t ld_dup,
                             int dtype, void* stream) {
  using namespace bt;
  BT_CHECK_ARG(rows >= 0 && cols >= 0, "swiglu_bwd: negative size");
  if (rows == 0 || cols == 0) return BT_OK;
  BT_CHECK_ARG(dy && gate && up && dgate && dup, "swiglu_bwd: null pointer");
  BT_CHECK_ARG(ld_dy >= cols && ld_gate >= cols && ld_up >= cols && ld_dgate >= cols &&
                   ld_dup >= cols,
               "swiglu_bwd: row stride smaller than cols");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case BT_BF16:
      return bwd_t<__nv_bfloat16>(dy, gate, up, dgate, dup, rows, cols, ld_dy, ld_gate, ld_up,
                                  ld_dgate, ld_dup, s);
    case BT_FP16:
      return bwd_t<__half>(dy, gate, up, dgate, dup, rows, cols, ld_dy, ld_gate, ld_up, ld_dgate,
                           ld_dup, s);
    case BT_FP32:
      return bwd_t<float>(dy, gate, up, dgate, dup, rows, cols, ld_dy, ld_gate, ld_up, ld_dgate,
                          ld_dup, s);
  }
  set_error("swiglu_bwd: unknown dtype %d", dtype);
  return BT_ERR_ARG;
}

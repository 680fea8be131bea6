// RMSNorm forward / backward for wide rows (a row no longer fits a few registers per
// lane): rows are streamed through shared memory by bulk asynchronous copies, so the
// bytes in flight per SM are set by the ring depth and not by the register file.
//
//   CTA = 256 threads, persistent over tiles of R rows.  A ring of S shared-memory
//   stages each holds one tile (forward: R rows of x; backward: R rows of x and dy).
//   Thread 0 arms a stage's mbarrier with the tile's byte count and issues one bulk
//   copy per row (rows may be strided in global memory); every thread then waits for
//   the stage (bounded wait), reads its fixed set of 16-byte column slices from shared
//   memory, and the row sums go through a small shared-memory reduction.  Because a
//   thread always owns the same columns, the backward keeps its slice of dw in
//   registers across all rows the CTA visits.
//
//   A stage is refilled right after the __syncthreads that ends its consumption, S-1
//   tiles ahead of use.
#pragma once

#include "bt_common.cuh"
#include "sm100_ptx.cuh"

namespace bt {

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

namespace staged {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kStages = 3;

// Set when a bounded wait for a bulk copy ran out (read back by bt_device_wait_errors).
__device__ int g_wait_error = 0;

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes,
                                          uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          ptx::smem_u32(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(ptx::smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ uint4 lds_v4(const void* p) { return *reinterpret_cast<const uint4*>(p); }

// Block-wide sums of R per-thread values; result in every thread.  `red` is [R][kWarps].
template <int R>
__device__ __forceinline__ void block_sums(float (&v)[R], float* red, int warp, int lane) {
#pragma unroll
  for (int r = 0; r < R; ++r) {
    v[r] = group_sum<32>(v[r]);
    if (lane == 0) red[r * kWarps + warp] = v[r];
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const float4 a = *reinterpret_cast<const float4*>(red + r * kWarps);
    const float4 b = *reinterpret_cast<const float4*>(red + r * kWarps + 4);
    v[r] = ((a.x + a.y) + (a.z + a.w)) + ((b.x + b.y) + (b.z + b.w));
  }
}

struct Ring {
  uint64_t full[kStages];
  int abort_flag;
};

// ------------------------------------------------------------------ forward
template <typename T, int VPT, int R>
__global__ void __launch_bounds__(kThreads, 2)
rms_fwd_staged(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
               float* __restrict__ rstd, int64_t M, int N, int64_t ld_x, int64_t ld_y, float eps) {
  constexpr int E = Cvt<T>::N;
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t row_bytes = static_cast<uint32_t>(N) * sizeof(T);
  const uint32_t stage_bytes = R * row_bytes;
  uint8_t* data = smem;
  float* red = reinterpret_cast<float*>(smem + kStages * stage_bytes);  // [2][R][kWarps]
  Ring* ring = reinterpret_cast<Ring*>(red + 2 * R * kWarps);
  const int nv = N / E;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float inv_n = 1.0f / static_cast<float>(N);
  const int64_t tiles = (M + R - 1) / R;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) ptx::mbar_init(&ring->full[s], 1);
    ring->abort_flag = 0;
    ptx::fence_mbar_init();
  }
  __syncthreads();

  auto issue = [&](int64_t tile, int s) {
    const int64_t r0 = tile * R;
    const int rows = static_cast<int>(M - r0 < R ? M - r0 : R);
    ptx::mbar_arrive_expect_tx(&ring->full[s], rows * row_bytes);
    for (int r = 0; r < rows; ++r)
      bulk_load(data + s * stage_bytes + r * row_bytes, x + (r0 + r) * ld_x, row_bytes,
                &ring->full[s]);
  };
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      const int64_t t = blockIdx.x + static_cast<int64_t>(s) * gridDim.x;
      if (t < tiles) issue(t, s);
    }
  }

  float wf[VPT][E];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * kThreads;
    Cvt<T>::unpack(v < nv ? ld_global_v4(w + static_cast<int64_t>(v) * E) : make_uint4(0, 0, 0, 0),
                   wf[i]);
  }

  int s = 0;
  uint32_t phase = 0;
  int buf = 0;
  for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    if (!ptx::mbar_wait(&ring->full[s], phase, &ring->abort_flag, &g_wait_error, 1)) break;
    const uint8_t* st = data + s * stage_bytes;
    const int64_t r0 = tile * R;
    float ss[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      ss[r] = 0.f;
      if (r0 + r < M) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int v = threadIdx.x + i * kThreads;
          if (v < nv) {
            float f[E];
            Cvt<T>::unpack(lds_v4(st + r * row_bytes + v * 16), f);
#pragma unroll
            for (int e = 0; e < E; ++e) ss[r] = fmaf(f[e], f[e], ss[r]);
          }
        }
      }
    }
    block_sums<R>(ss, red + buf * R * kWarps, warp, lane);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int64_t row = r0 + r;
      if (row < M) {
        const float rs = rsqrtf(ss[r] * inv_n + eps);
        if (threadIdx.x == 0) rstd[row] = rs;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int v = threadIdx.x + i * kThreads;
          if (v < nv) {
            float f[E];
            Cvt<T>::unpack(lds_v4(st + r * row_bytes + v * 16), f);
#pragma unroll
            for (int e = 0; e < E; ++e) f[e] = f[e] * rs * wf[i][e];
            st_global_v4(y + row * ld_y + static_cast<int64_t>(v) * E, Cvt<T>::pack(f));
          }
        }
      }
    }
    __syncthreads();  // everyone is done with stage s
    if (threadIdx.x == 0) {
      const int64_t nt = tile + static_cast<int64_t>(kStages) * gridDim.x;
      if (nt < tiles) issue(nt, s);
    }
    buf ^= 1;
    if (++s == kStages) {
      s = 0;
      phase ^= 1u;
    }
  }
}

// ----------------------------------------------------------------- backward
// ws: dw_copies(N) x N fp32 column sums + arrival counter, zero on entry, left zero on exit.
template <typename T, int VPT, int R>
__global__ void __launch_bounds__(kThreads, 2)
rms_bwd_staged(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
               const float* __restrict__ rstd, T* __restrict__ dx, T* __restrict__ dw,
               float* __restrict__ ws, int64_t M, int N, int64_t ld_dy, int64_t ld_x,
               int64_t ld_dx) {
  constexpr int E = Cvt<T>::N;
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t row_bytes = static_cast<uint32_t>(N) * sizeof(T);
  const uint32_t stage_bytes = 2 * R * row_bytes;  // R rows of x, then R rows of dy
  uint8_t* data = smem;
  float* red = reinterpret_cast<float*>(smem + kStages * stage_bytes);
  Ring* ring = reinterpret_cast<Ring*>(red + 2 * R * kWarps);
  const int nv = N / E;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float inv_n = 1.0f / static_cast<float>(N);
  const int64_t tiles = (M + R - 1) / R;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) ptx::mbar_init(&ring->full[s], 1);
    ring->abort_flag = 0;
    ptx::fence_mbar_init();
  }
  __syncthreads();

  auto issue = [&](int64_t tile, int s) {
    const int64_t r0 = tile * R;
    const int rows = static_cast<int>(M - r0 < R ? M - r0 : R);
    ptx::mbar_arrive_expect_tx(&ring->full[s], 2 * rows * row_bytes);
    uint8_t* base = data + s * stage_bytes;
    for (int r = 0; r < rows; ++r) {
      bulk_load(base + r * row_bytes, x + (r0 + r) * ld_x, row_bytes, &ring->full[s]);
      bulk_load(base + (R + r) * row_bytes, dy + (r0 + r) * ld_dy, row_bytes, &ring->full[s]);
    }
  };
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      const int64_t t = blockIdx.x + static_cast<int64_t>(s) * gridDim.x;
      if (t < tiles) issue(t, s);
    }
  }

  float wf[VPT][E], acc[VPT][E];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * kThreads;
    Cvt<T>::unpack(v < nv ? ld_global_v4(w + static_cast<int64_t>(v) * E) : make_uint4(0, 0, 0, 0),
                   wf[i]);
#pragma unroll
    for (int e = 0; e < E; ++e) acc[i][e] = 0.f;
  }

  int s = 0;
  uint32_t phase = 0;
  int buf = 0;
  for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    if (!ptx::mbar_wait(&ring->full[s], phase, &ring->abort_flag, &g_wait_error, 2)) break;
    const uint8_t* sx = data + s * stage_bytes;
    const uint8_t* sg = sx + R * row_bytes;
    const int64_t r0 = tile * R;
    float dot[R], rs[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      dot[r] = 0.f;
      rs[r] = (r0 + r < M) ? rstd[r0 + r] : 0.f;
      if (r0 + r < M) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int v = threadIdx.x + i * kThreads;
          if (v < nv) {
            float xf[E], gf[E];
            Cvt<T>::unpack(lds_v4(sx + r * row_bytes + v * 16), xf);
            Cvt<T>::unpack(lds_v4(sg + r * row_bytes + v * 16), gf);
#pragma unroll
            for (int e = 0; e < E; ++e) {
              const float xh = xf[e] * rs[r];
              dot[r] = fmaf(xh, gf[e] * wf[i][e], dot[r]);
              acc[i][e] = fmaf(gf[e], xh, acc[i][e]);
            }
          }
        }
      }
    }
    block_sums<R>(dot, red + buf * R * kWarps, warp, lane);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int64_t row = r0 + r;
      if (row < M) {
        const float c = dot[r] * inv_n;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int v = threadIdx.x + i * kThreads;
          if (v < nv) {
            float xf[E], gf[E], o[E];
            Cvt<T>::unpack(lds_v4(sx + r * row_bytes + v * 16), xf);
            Cvt<T>::unpack(lds_v4(sg + r * row_bytes + v * 16), gf);
#pragma unroll
            for (int e = 0; e < E; ++e) o[e] = (gf[e] * wf[i][e] - xf[e] * rs[r] * c) * rs[r];
            st_global_v4(dx + row * ld_dx + static_cast<int64_t>(v) * E, Cvt<T>::pack(o));
          }
        }
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      const int64_t nt = tile + static_cast<int64_t>(kStages) * gridDim.x;
      if (nt < tiles) issue(nt, s);
    }
    buf ^= 1;
    if (++s == kStages) {
      s = 0;
      phase ^= 1u;
    }
  }

  const int K = dw_copies(N);
  {
    float* my_ws = ws + static_cast<int64_t>(blockIdx.x % K) * N;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = threadIdx.x + i * kThreads;
      if (v < nv) {
#pragma unroll
        for (int e = 0; e < E; e += 4)
          red_add_v4(my_ws + v * E + e, acc[i][e], acc[i][e + 1], acc[i][e + 2], acc[i][e + 3]);
      }
    }
  }
  dw_finalize<T>(ws, dw, N, gridDim.x, threadIdx.x, kThreads);
}

inline size_t smem_bytes(int N, int elem, int R, bool bwd) {
  return static_cast<size_t>(kStages) * (bwd ? 2 : 1) * R * N * elem + 2 * R * kWarps * sizeof(float) +
         sizeof(Ring) + 16;
}

}  // namespace staged
}  // namespace bt

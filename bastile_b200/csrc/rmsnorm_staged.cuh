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
// ADD: a stage holds R rows of x and R rows of the residual; the rounded sum replaces x in
// shared memory (a thread only ever touches its own column slices), is written to `sum`,
// and is what gets normalised.
template <typename T, int VPT, int R, bool ADD>
__global__ void __launch_bounds__(kThreads, 2)
rms_fwd_staged(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
               float* __restrict__ rstd, int64_t M, int N, int64_t ld_x, int64_t ld_y, float eps,
               const T* __restrict__ res, T* __restrict__ sum, int64_t ld_res, int64_t ld_sum) {
  constexpr int E = Cvt<T>::N;
  constexpr int kArrays = ADD ? 2 : 1;
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t row_bytes = static_cast<uint32_t>(N) * sizeof(T);
  const uint32_t stage_bytes = kArrays * R * row_bytes;
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
  grid_dependency_wait();  // everything above ran while the previous kernel of the stream drained

  auto issue = [&](int64_t tile, int s) {
    const int64_t r0 = tile * R;
    const int rows = static_cast<int>(M - r0 < R ? M - r0 : R);
    ptx::mbar_arrive_expect_tx(&ring->full[s], kArrays * rows * row_bytes);
    uint8_t* base = data + s * stage_bytes;
    for (int r = 0; r < rows; ++r) {
      bulk_load(base + r * row_bytes, x + (r0 + r) * ld_x, row_bytes, &ring->full[s]);
      if constexpr (ADD)
        bulk_load(base + (R + r) * row_bytes, res + (r0 + r) * ld_res, row_bytes, &ring->full[s]);
    }
  };
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      const int64_t t = blockIdx.x + static_cast<int64_t>(s) * gridDim.x;
      if (t < tiles) issue(t, s);
    }
  }

  constexpr int P = E / 2;  // fp32 pairs per 16-byte vector
  f32x2 wf[VPT][P];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * kThreads;
    unpack_pairs<T>(v < nv ? ld_global_v4(w + static_cast<int64_t>(v) * E) : make_uint4(0, 0, 0, 0),
                    wf[i]);
  }

  int s = 0;
  uint32_t phase = 0;
  int buf = 0;
  for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    // A thread whose wait ran out (or that saw another thread give up) does not leave by itself:
    // it skips the arithmetic, joins the block-wide sum below, and after that barrier EVERY thread
    // reads the same abort flag and leaves together - no thread is ever left alone at a barrier.
    const bool ok = ptx::mbar_wait(&ring->full[s], phase, &ring->abort_flag, &g_wait_error, 1);
    uint8_t* st = data + s * stage_bytes;
    const int64_t r0 = tile * R;
    float ss[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      f32x2 ss2 = pair(0.f, 0.f);  // even / odd elements of this thread's slices
      if (ok && r0 + r < M) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int v = threadIdx.x + i * kThreads;
          if (v < nv) {
            f32x2 f[P];
            if constexpr (ADD) {
              f32x2 b[P];
              unpack_pairs<T>(lds_v4(st + r * row_bytes + v * 16), f);
              unpack_pairs<T>(lds_v4(st + (R + r) * row_bytes + v * 16), b);
#pragma unroll
              for (int e = 0; e < P; ++e) f[e] = add2(f[e], b[e]);
              const uint4 packed = pack_pairs<T>(f);
              *reinterpret_cast<uint4*>(st + r * row_bytes + v * 16) = packed;
              st_global_v4(sum + (r0 + r) * ld_sum + static_cast<int64_t>(v) * E, packed);
              unpack_pairs<T>(packed, f);
            } else {
              unpack_pairs<T>(lds_v4(st + r * row_bytes + v * 16), f);
            }
#pragma unroll
            for (int e = 0; e < P; ++e) ss2 = fma2(f[e], f[e], ss2);
          }
        }
      }
      ss[r] = lo_of(ss2) + hi_of(ss2);
    }
    block_sums<R>(ss, red + buf * R * kWarps, warp, lane);
    if (*reinterpret_cast<volatile int*>(&ring->abort_flag) != 0) break;  // same value in every thread
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int64_t row = r0 + r;
      if (row < M) {
        const float rs = rsqrtf(ss[r] * inv_n + eps);
        if (threadIdx.x == 0) rstd[row] = rs;
        const f32x2 rs2 = pair(rs, rs);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int v = threadIdx.x + i * kThreads;
          if (v < nv) {
            f32x2 f[P];
            unpack_pairs<T>(lds_v4(st + r * row_bytes + v * 16), f);
#pragma unroll
            for (int e = 0; e < P; ++e) f[e] = mul2(mul2(f[e], rs2), wf[i][e]);
            st_global_v4(y + row * ld_y + static_cast<int64_t>(v) * E, pack_pairs<T>(f));
          }
        }
      }
    }
    if constexpr (ADD) ptx::fence_proxy_async_smem();  // our stores before the refill's writes
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
// ADD: dx also takes in `dres`, the gradient arriving along the residual path; its slices
// are fetched straight into registers at the top of a tile, ahead of the first pass.
template <typename T, int VPT, int R, bool ADD>
__global__ void __launch_bounds__(kThreads, 2)
rms_bwd_staged(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
               const float* __restrict__ rstd, T* __restrict__ dx, T* __restrict__ dw,
               float* __restrict__ ws, int64_t M, int N, int64_t ld_dy, int64_t ld_x,
               int64_t ld_dx, const T* __restrict__ dres, int64_t ld_dres) {
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
  grid_dependency_wait();  // everything above ran while the previous kernel of the stream drained

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

  constexpr int P = E / 2;  // fp32 pairs per 16-byte vector
  f32x2 wf[VPT][P], acc[VPT][P];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * kThreads;
    unpack_pairs<T>(v < nv ? ld_global_v4(w + static_cast<int64_t>(v) * E) : make_uint4(0, 0, 0, 0),
                    wf[i]);
#pragma unroll
    for (int e = 0; e < P; ++e) acc[i][e] = pair(0.f, 0.f);
  }

  int s = 0;
  uint32_t phase = 0;
  int buf = 0;
  for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const int64_t r0 = tile * R;
    uint4 rv[ADD ? R : 1][ADD ? VPT : 1];
    if constexpr (ADD) {
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int v = threadIdx.x + i * kThreads;
          rv[r][i] = (r0 + r < M && v < nv)
                         ? ld_stream_v4(dres + (r0 + r) * ld_dres + static_cast<int64_t>(v) * E)
                         : make_uint4(0, 0, 0, 0);
        }
    }
    // as in the forward: nobody leaves before the barrier inside block_sums, everybody after it
    const bool ok = ptx::mbar_wait(&ring->full[s], phase, &ring->abort_flag, &g_wait_error, 2);
    const uint8_t* sx = data + s * stage_bytes;
    const uint8_t* sg = sx + R * row_bytes;
    float dot[R], rs[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      f32x2 dot2 = pair(0.f, 0.f);
      rs[r] = (r0 + r < M) ? rstd[r0 + r] : 0.f;
      const f32x2 rs2 = pair(rs[r], rs[r]);
      if (ok && r0 + r < M) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int v = threadIdx.x + i * kThreads;
          if (v < nv) {
            f32x2 xf[P], gf[P];
            unpack_pairs<T>(lds_v4(sx + r * row_bytes + v * 16), xf);
            unpack_pairs<T>(lds_v4(sg + r * row_bytes + v * 16), gf);
#pragma unroll
            for (int e = 0; e < P; ++e) {
              const f32x2 xh = mul2(xf[e], rs2);
              dot2 = fma2(xh, mul2(gf[e], wf[i][e]), dot2);
              acc[i][e] = fma2(gf[e], xh, acc[i][e]);
            }
          }
        }
      }
      dot[r] = lo_of(dot2) + hi_of(dot2);
    }
    block_sums<R>(dot, red + buf * R * kWarps, warp, lane);
    if (*reinterpret_cast<volatile int*>(&ring->abort_flag) != 0) break;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int64_t row = r0 + r;
      if (row < M) {
        const float c = dot[r] * inv_n;
        const f32x2 rs2 = pair(rs[r], rs[r]);
        const f32x2 neg_rs_c = pair(-rs[r] * c, -rs[r] * c);  // (g*w - x*rs*c)*rs = (g*w + x*(-rs*c))*rs
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int v = threadIdx.x + i * kThreads;
          if (v < nv) {
            f32x2 xf[P], gf[P], o[P];
            unpack_pairs<T>(lds_v4(sx + r * row_bytes + v * 16), xf);
            unpack_pairs<T>(lds_v4(sg + r * row_bytes + v * 16), gf);
#pragma unroll
            for (int e = 0; e < P; ++e) o[e] = mul2(fma2(xf[e], neg_rs_c, mul2(gf[e], wf[i][e])), rs2);
            if constexpr (ADD) {
              f32x2 a[P];
              unpack_pairs<T>(rv[r][i], a);
#pragma unroll
              for (int e = 0; e < P; ++e) o[e] = add2(o[e], a[e]);
            }
            st_global_v4(dx + row * ld_dx + static_cast<int64_t>(v) * E, pack_pairs<T>(o));
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
        for (int e = 0; e < P; e += 2)
          red_add_v4(my_ws + v * E + 2 * e, lo_of(acc[i][e]), hi_of(acc[i][e]), lo_of(acc[i][e + 1]),
                     hi_of(acc[i][e + 1]));
      }
    }
  }
  dw_finalize<T>(ws, dw, N, gridDim.x, threadIdx.x, kThreads);
}

// `arrays`: row sets per stage (forward: x [+ residual]; backward: x and dy).
inline size_t smem_bytes(int N, int elem, int R, int arrays) {
  return static_cast<size_t>(kStages) * arrays * R * N * elem + 2 * R * kWarps * sizeof(float) +
         sizeof(Ring) + 16;
}

}  // namespace staged
}  // namespace bt

// RMSNorm forward / backward for sm_100a: bandwidth-bound, every row is read
// from HBM exactly once and kept in registers between the reduction and the
// scaled write-back.
//
// Layouts
//   rows kernel  : (rows of up to 2 KB, e.g. the 128-wide q/k norms) a group of LPR
//                  lanes (8..32) owns one row, VPT 16-byte vectors per lane in
//                  registers; a 256-thread CTA works on 256/LPR rows x RPI at a
//                  time.  Row sums are warp shuffles only.
//   staged kernel: (rows of 2..16 KB, e.g. hidden 4096) rows stream through a
//                  shared-memory ring filled by bulk asynchronous copies
//                  (rmsnorm_staged.cuh).
//   generic      : any N / alignment, scalar accesses; correctness net only.
//
// dw is accumulated as fp32 partial sums: registers -> shared -> one global
// atomic per column per CTA into a zeroed scratch row; the last CTA to finish
// converts the row to the weight dtype and zeroes the scratch again.
#include <mutex>

#include "bt_common.cuh"
#include "rmsnorm_staged.cuh"

namespace bt {
namespace {

constexpr int kThreads = 256;

// ------------------------------------------------------------------ forward
// ADD: the row that is normalised is T(x + res); it is also written to `sum`.
template <typename T, int VPT, int LPR, int RPI, bool ADD>
__global__ void __launch_bounds__(kThreads, (VPT >= 16 ? 2 : (VPT >= 8 ? 3 : 4)))
rms_fwd_rows(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
             float* __restrict__ rstd, int64_t M, int N, int64_t ld_x, int64_t ld_y, float eps,
             const T* __restrict__ res, T* __restrict__ sum, int64_t ld_res, int64_t ld_sum) {
  constexpr int E = Cvt<T>::N;
  constexpr int kGroups = kThreads / LPR;
  const int lane = threadIdx.x % LPR;
  const int group = threadIdx.x / LPR;
  const int nv = N / E;
  const float inv_n = 1.0f / static_cast<float>(N);
  const int64_t rows_per_iter = static_cast<int64_t>(kGroups) * RPI;
  grid_dependency_wait();

  for (int64_t base = static_cast<int64_t>(blockIdx.x) * rows_per_iter; base < M;
       base += static_cast<int64_t>(gridDim.x) * rows_per_iter) {
    uint4 xv[RPI][VPT];
#pragma unroll
    for (int r = 0; r < RPI; ++r) {
      const int64_t row = base + r * kGroups + group;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = lane + i * LPR;
        xv[r][i] = (row < M && v < nv) ? ld_stream_v4(x + row * ld_x + static_cast<int64_t>(v) * E)
                                       : make_uint4(0, 0, 0, 0);
      }
    }
    if constexpr (ADD) {
      uint4 rv[RPI][VPT];
#pragma unroll
      for (int r = 0; r < RPI; ++r) {
        const int64_t row = base + r * kGroups + group;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int v = lane + i * LPR;
          rv[r][i] = (row < M && v < nv)
                         ? ld_stream_v4(res + row * ld_res + static_cast<int64_t>(v) * E)
                         : make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int r = 0; r < RPI; ++r) {
        const int64_t row = base + r * kGroups + group;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int v = lane + i * LPR;
          float a[E], b[E];
          Cvt<T>::unpack(xv[r][i], a);
          Cvt<T>::unpack(rv[r][i], b);
#pragma unroll
          for (int e = 0; e < E; ++e) a[e] += b[e];
          xv[r][i] = Cvt<T>::pack(a);
          if (row < M && v < nv)
            st_global_v4(sum + row * ld_sum + static_cast<int64_t>(v) * E, xv[r][i]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < RPI; ++r) {
      const int64_t row = base + r * kGroups + group;
      float ss = 0.f;  // one scalar chain, element by element: its order is pinned by tests
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        float f[E];
        Cvt<T>::unpack(xv[r][i], f);
#pragma unroll
        for (int e = 0; e < E; ++e) ss = fmaf(f[e], f[e], ss);
      }
      ss = group_sum<LPR>(ss);
      const float rs = rsqrtf(ss * inv_n + eps);
#pragma unroll
      for (int i = 0; i < VPT; ++i) forget_unpacked(xv[r][i]);
      if (row < M) {
        if (lane == 0) rstd[row] = rs;
        const f32x2 rs2 = pair(rs, rs);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int v = lane + i * LPR;
          if (v < nv) {
            // elementwise part on packed fp32 pairs: same value per element, half the issue slots
            f32x2 f[E / 2], wf[E / 2];
            unpack_pairs<T>(xv[r][i], f);
            unpack_pairs<T>(ld_global_v4(w + static_cast<int64_t>(v) * E), wf);
#pragma unroll
            for (int e = 0; e < E / 2; ++e) f[e] = mul2(mul2(f[e], rs2), wf[e]);
            st_global_v4(y + row * ld_y + static_cast<int64_t>(v) * E, pack_pairs<T>(f));
          }
        }
      }
    }
  }
}

// One CTA per row, scalar accesses, two passes (second one from cache).
template <typename T>
__global__ void __launch_bounds__(kThreads)
rms_fwd_generic(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
                float* __restrict__ rstd, int64_t M, int64_t N, int64_t ld_x, int64_t ld_y,
                float eps, const T* __restrict__ res, T* sum, int64_t ld_res, int64_t ld_sum) {
  __shared__ float red[kThreads / 32];
  __shared__ float s_rs;
  for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
    const T* xr = x + row * ld_x;
    float ss = 0.f;
    if (res != nullptr) {
      // each thread writes and later re-reads its own columns of the summed row
      T* sr = sum + row * ld_sum;
      for (int64_t c = threadIdx.x; c < N; c += kThreads) {
        const T t = Cvt<T>::from_f(Cvt<T>::to_f(xr[c]) + Cvt<T>::to_f(res[row * ld_res + c]));
        sr[c] = t;
        const float f = Cvt<T>::to_f(t);
        ss = fmaf(f, f, ss);
      }
      xr = sr;
    } else {
      for (int64_t c = threadIdx.x; c < N; c += kThreads) {
        const float f = Cvt<T>::to_f(xr[c]);
        ss = fmaf(f, f, ss);
      }
    }
    ss = group_sum<32>(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int i = 0; i < kThreads / 32; ++i) t += red[i];
      s_rs = rsqrtf(t / static_cast<float>(N) + eps);
      rstd[row] = s_rs;
    }
    __syncthreads();
    const float rs = s_rs;
    for (int64_t c = threadIdx.x; c < N; c += kThreads)
      y[row * ld_y + c] = Cvt<T>::from_f(Cvt<T>::to_f(xr[c]) * rs * Cvt<T>::to_f(w[c]));
    __syncthreads();
  }
}

// ----------------------------------------------------------------- backward
// Scratch layout: dw_copies(N) x float acc[N], then one uint32 arrival counter.
// ADD: dx = T(norm backward + dres), dres read where dx is written.
template <typename T, int VPT, int LPR, int RPI, bool ADD>
__global__ void __launch_bounds__(kThreads, 3)
rms_bwd_rows(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
             const float* __restrict__ rstd, T* __restrict__ dx, T* __restrict__ dw,
             float* __restrict__ ws, int64_t M, int N, int64_t ld_dy, int64_t ld_x,
             int64_t ld_dx, const T* __restrict__ dres, int64_t ld_dres) {
  constexpr int E = Cvt<T>::N;
  constexpr int kGroups = kThreads / LPR;
  extern __shared__ float s_dw[];  // N floats
  const int lane = threadIdx.x % LPR;
  const int group = threadIdx.x / LPR;
  const int nv = N / E;
  const float inv_n = 1.0f / static_cast<float>(N);
  const int64_t rows_per_iter = static_cast<int64_t>(kGroups) * RPI;

  for (int c = threadIdx.x; c < N; c += kThreads) s_dw[c] = 0.f;
  grid_dependency_wait();

  // elementwise arithmetic on packed fp32 pairs (half the issue slots, same values); the dot
  // product stays one scalar chain, whose order is pinned by tests
  constexpr int P = E / 2;
  f32x2 wf[VPT][P];
  f32x2 acc[VPT][P];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = lane + i * LPR;
    uint4 wv = (v < nv) ? ld_global_v4(w + static_cast<int64_t>(v) * E) : make_uint4(0, 0, 0, 0);
    unpack_pairs<T>(wv, wf[i]);
#pragma unroll
    for (int e = 0; e < P; ++e) acc[i][e] = pair(0.f, 0.f);
  }

  for (int64_t base = static_cast<int64_t>(blockIdx.x) * rows_per_iter; base < M;
       base += static_cast<int64_t>(gridDim.x) * rows_per_iter) {
    uint4 xv[RPI][VPT], gv[RPI][VPT];
    float rs[RPI];
#pragma unroll
    for (int r = 0; r < RPI; ++r) {
      const int64_t row = base + r * kGroups + group;
      rs[r] = (row < M) ? rstd[row] : 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = lane + i * LPR;
        const bool ok = (row < M && v < nv);
        xv[r][i] = ok ? ld_stream_v4(x + row * ld_x + static_cast<int64_t>(v) * E)
                      : make_uint4(0, 0, 0, 0);
        gv[r][i] = ok ? ld_stream_v4(dy + row * ld_dy + static_cast<int64_t>(v) * E)
                      : make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int r = 0; r < RPI; ++r) {
      const int64_t row = base + r * kGroups + group;
      float dot = 0.f;
      const f32x2 rs2 = pair(rs[r], rs[r]);
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        f32x2 xf[P], gf[P];
        unpack_pairs<T>(xv[r][i], xf);
        unpack_pairs<T>(gv[r][i], gf);
#pragma unroll
        for (int e = 0; e < P; ++e) {
          const f32x2 xh = mul2(xf[e], rs2);
          const f32x2 t = mul2(gf[e], wf[i][e]);
          dot = fmaf(lo_of(xh), lo_of(t), dot);
          dot = fmaf(hi_of(xh), hi_of(t), dot);
          acc[i][e] = fma2(gf[e], xh, acc[i][e]);
        }
      }
      dot = group_sum<LPR>(dot) * inv_n;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        forget_unpacked(xv[r][i]);
        forget_unpacked(gv[r][i]);
      }
      if (row < M) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int v = lane + i * LPR;
          if (v < nv) {
            f32x2 xf[P], gf[P], o[P];
            unpack_pairs<T>(xv[r][i], xf);
            unpack_pairs<T>(gv[r][i], gf);
            const f32x2 ndot = pair(-dot, -dot);
#pragma unroll
            for (int e = 0; e < P; ++e)  // explicit operations: the fused q/k-norm + RoPE backward
              // spells out the same ones and stays bit-identical: fma(-(x*rs), dot, g*w) * rs
              o[e] = mul2(fma2(mul2(xf[e], rs2), ndot, mul2(gf[e], wf[i][e])), rs2);
            if constexpr (ADD) {
              f32x2 a[P];
              unpack_pairs<T>(ld_stream_v4(dres + row * ld_dres + static_cast<int64_t>(v) * E), a);
#pragma unroll
              for (int e = 0; e < P; ++e) o[e] = add2(o[e], a[e]);
            }
            st_global_v4(dx + row * ld_dx + static_cast<int64_t>(v) * E, pack_pairs<T>(o));
          }
        }
      }
    }
  }

  __syncthreads();  // s_dw zeroed
  // Row groups that share a warp hold the same columns: fold them together first.
  float accf[VPT][E];
#pragma unroll
  for (int i = 0; i < VPT; ++i)
#pragma unroll
    for (int e = 0; e < P; ++e) {
      accf[i][2 * e] = lo_of(acc[i][e]);
      accf[i][2 * e + 1] = hi_of(acc[i][e]);
    }
#pragma unroll
  for (int o = LPR; o < 32; o <<= 1) {
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int e = 0; e < E; ++e) accf[i][e] += __shfl_xor_sync(0xffffffffu, accf[i][e], o);
  }
  // s_dw is kept element-major (index e * nv + v) so that the lanes of one instruction,
  // which differ in v, fall into different banks.
  if ((threadIdx.x & 31) < LPR) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = lane + i * LPR;
      if (v < nv) {
#pragma unroll
        for (int e = 0; e < E; ++e) atomicAdd(&s_dw[e * nv + v], accf[i][e]);
      }
    }
  }
  __syncthreads();
  float* my_ws = ws + static_cast<int64_t>(blockIdx.x % dw_copies(N)) * N;
  for (int c = threadIdx.x; c < N; c += kThreads) atomicAdd(my_ws + c, s_dw[(c % E) * nv + c / E]);
  dw_finalize<T>(ws, dw, N, gridDim.x, threadIdx.x, kThreads);
}

// Generic backward, part 1: dx, one CTA per row (scalar).
template <typename T>
__global__ void __launch_bounds__(kThreads)
rms_bwd_dx_generic(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
                   const float* __restrict__ rstd, T* __restrict__ dx, int64_t M, int64_t N,
                   int64_t ld_dy, int64_t ld_x, int64_t ld_dx, const T* __restrict__ dres,
                   int64_t ld_dres) {
  __shared__ float red[kThreads / 32];
  __shared__ float s_dot;
  for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
    const float rs = rstd[row];
    float d = 0.f;
    for (int64_t c = threadIdx.x; c < N; c += kThreads)
      d = fmaf(Cvt<T>::to_f(x[row * ld_x + c]) * rs,
               Cvt<T>::to_f(dy[row * ld_dy + c]) * Cvt<T>::to_f(w[c]), d);
    d = group_sum<32>(d);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = d;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int i = 0; i < kThreads / 32; ++i) t += red[i];
      s_dot = t / static_cast<float>(N);
    }
    __syncthreads();
    const float dot = s_dot;
    for (int64_t c = threadIdx.x; c < N; c += kThreads) {
      const float xh = Cvt<T>::to_f(x[row * ld_x + c]) * rs;
      const float wdy = Cvt<T>::to_f(dy[row * ld_dy + c]) * Cvt<T>::to_f(w[c]);
      float o = (wdy - xh * dot) * rs;
      if (dres != nullptr) o += Cvt<T>::to_f(dres[row * ld_dres + c]);
      dx[row * ld_dx + c] = Cvt<T>::from_f(o);
    }
    __syncthreads();
  }
}

// Generic backward, part 2: dw.  blockDim = (32 columns, 8 row lanes).
template <typename T>
__global__ void rms_bwd_dw_generic(const T* __restrict__ dy, const T* __restrict__ x,
                                   const float* __restrict__ rstd, T* __restrict__ dw,
                                   float* __restrict__ ws, int64_t M, int N, int64_t ld_dy,
                                   int64_t ld_x) {
  const int c = blockIdx.x * 32 + threadIdx.x;
  float a = 0.f;
  if (c < N) {
    for (int64_t row = static_cast<int64_t>(blockIdx.y) * blockDim.y + threadIdx.y; row < M;
         row += static_cast<int64_t>(gridDim.y) * blockDim.y)
      a = fmaf(Cvt<T>::to_f(dy[row * ld_dy + c]), Cvt<T>::to_f(x[row * ld_x + c]) * rstd[row], a);
    atomicAdd(ws + static_cast<int64_t>(blockIdx.y % dw_copies(N)) * N + c, a);
  }
  dw_finalize<T>(ws, dw, N, gridDim.x * gridDim.y, threadIdx.y * 32 + threadIdx.x, 32 * blockDim.y);
}

// ------------------------------------------------------------ host dispatch
struct RowCfg {
  int lpr, vpt, rpi;
};

// nv = 16-byte vectors per row.  Returns false when the rows layout does not apply.
bool pick_rows(int64_t nv, int max_vpt, RowCfg* c) {
  if (nv <= 0) return false;
  int lpr = 8;
  while (lpr < 32 && lpr < nv) lpr *= 2;
  int vpt = 1;
  while (static_cast<int64_t>(vpt) * lpr < nv) vpt *= 2;
  if (vpt > max_vpt) return false;
  c->lpr = lpr;
  c->vpt = vpt;
  c->rpi = (vpt == 1) ? 4 : (vpt == 2 ? 2 : 1);
  return true;
}

int grid_for(int64_t work_items, int ctas_per_sm) {
  const int64_t cap = static_cast<int64_t>(sm_count()) * ctas_per_sm;
  return static_cast<int>(work_items < cap ? (work_items < 1 ? 1 : work_items) : cap);
}

// Optional residual operands of the fused add + norm entry points (all null for the plain ones).
struct Residual {
  const void* res = nullptr;   // forward: added to x before the norm
  void* sum = nullptr;         // forward: T(x + res)
  int64_t ld_res = 0, ld_sum = 0;
  const void* dres = nullptr;  // backward: added to dx
  int64_t ld_dres = 0;
};

template <typename T, bool ADD>
int fwd_t(const void* x, const void* w, void* y, float* rstd, int64_t M, int64_t N, int64_t ld_x,
          int64_t ld_y, float eps, const Residual& rr, cudaStream_t s) {
  constexpr int E = Cvt<T>::N;
  const T* xp = static_cast<const T*>(x);
  const T* wp = static_cast<const T*>(w);
  T* yp = static_cast<T*>(y);
  const T* rp = static_cast<const T*>(rr.res);
  T* sp = static_cast<T*>(rr.sum);
  RowCfg c{};
  bool vec_ok = (N % E == 0) && (ld_x % E == 0) && (ld_y % E == 0) && aligned16(x) &&
                aligned16(w) && aligned16(y);
  if (ADD)
    vec_ok = vec_ok && (rr.ld_res % E == 0) && (rr.ld_sum % E == 0) && aligned16(rr.res) &&
             aligned16(rr.sum);
  const bool staged_ok = vec_ok && N / E > 128 && N / E <= 4 * staged::kThreads;
  if (!vec_ok || (!staged_ok && !pick_rows(N / E, 4, &c))) {
    rms_fwd_generic<T><<<grid_for(M, 8), kThreads, 0, s>>>(xp, wp, yp, rstd, M, N, ld_x, ld_y, eps,
                                                           rp, sp, rr.ld_res, rr.ld_sum);
    BT_CHECK_LAUNCH("rms_fwd_generic");
    return BT_OK;
  }
  if (staged_ok) {
    const int64_t nv = N / E;
    const int vpt = nv <= staged::kThreads ? 1 : (nv <= 2 * staged::kThreads ? 2 : 4);
    // a stage of the fused form holds twice the rows, so it takes half as many per tile
#define BT_FWDS(V, R0)                                                                           \
  if (vpt == V) {                                                                                \
    constexpr int R = ADD ? R0 / 2 : R0;                                                         \
    static const cudaError_t attr =                                                              \
        cudaFuncSetAttribute(staged::rms_fwd_staged<T, V, R, ADD>,                               \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);           \
    (void)attr;                                                                                  \
    const size_t smem = staged::smem_bytes(static_cast<int>(N), sizeof(T), R, ADD ? 2 : 1);      \
    const int grid = grid_for(ceil_div(M, R), 2);                                                \
    BT_CHECK_LAUNCHED(launch_dependent(staged::rms_fwd_staged<T, V, R, ADD>, dim3(grid),          \
                                       dim3(staged::kThreads), smem, s, xp, wp, yp, rstd, M,     \
                                       static_cast<int>(N), ld_x, ld_y, eps, rp, sp, rr.ld_res,  \
                                       rr.ld_sum),                                               \
                      "rms_fwd_staged");                                                         \
    return BT_OK;                                                                                \
  }
    BT_FWDS(1, 8)
    BT_FWDS(2, 4)
    BT_FWDS(4, 2)
#undef BT_FWDS
  }
  const int64_t rows_per_iter = static_cast<int64_t>(kThreads / c.lpr) * c.rpi;
  // many short-lived CTAs: the hardware scheduler evens out the tail better than a fixed split
  const int grid = grid_for(ceil_div(M, rows_per_iter), 32);
#define BT_FWD(L, V, R)                                                                        \
  if (c.lpr == L && c.vpt == V) {                                                              \
    BT_CHECK_LAUNCHED(launch_dependent(rms_fwd_rows<T, V, L, R, ADD>, dim3(grid), dim3(kThreads), \
                                       0, s, xp, wp, yp, rstd, M, static_cast<int>(N), ld_x,   \
                                       ld_y, eps, rp, sp, rr.ld_res, rr.ld_sum),               \
                      "rms_fwd_rows");                                                         \
    return BT_OK;                                                                              \
  }
  BT_FWD(8, 1, 4)
  BT_FWD(16, 1, 4)
  BT_FWD(32, 1, 4)
  BT_FWD(32, 2, 2)
  BT_FWD(32, 4, 1)
#undef BT_FWD
  set_error("rmsnorm_fwd: no kernel for lpr=%d vpt=%d", c.lpr, c.vpt);
  return BT_ERR_ARG;
}

template <typename T, bool ADD>
int bwd_t(const void* dy, const void* x, const void* w, const float* rstd, void* dx, void* dw,
          void* ws, int64_t M, int64_t N, int64_t ld_dy, int64_t ld_x, int64_t ld_dx,
          const Residual& rr, cudaStream_t s) {
  constexpr int E = Cvt<T>::N;
  const T* gp = static_cast<const T*>(dy);
  const T* xp = static_cast<const T*>(x);
  const T* wp = static_cast<const T*>(w);
  const T* rp = static_cast<const T*>(rr.dres);
  T* dxp = static_cast<T*>(dx);
  T* dwp = static_cast<T*>(dw);
  float* wsp = static_cast<float*>(ws);
  bool vec_ok = (N % E == 0) && (ld_x % E == 0) && (ld_dy % E == 0) && (ld_dx % E == 0) &&
                aligned16(x) && aligned16(w) && aligned16(dy) && aligned16(dx);
  if (ADD) vec_ok = vec_ok && (rr.ld_dres % E == 0) && aligned16(rr.dres);
  const int64_t nv = vec_ok ? N / E : 0;
  RowCfg c{};
  if (vec_ok && nv > 128 && nv <= 4 * staged::kThreads) {
    const int vpt = nv <= staged::kThreads ? 1 : (nv <= 2 * staged::kThreads ? 2 : 4);
#define BT_BWDS(V, R)                                                                            \
  if (vpt == V) {                                                                                \
    static const cudaError_t attr =                                                              \
        cudaFuncSetAttribute(staged::rms_bwd_staged<T, V, R, ADD>,                               \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);           \
    (void)attr;                                                                                  \
    const size_t smem = staged::smem_bytes(static_cast<int>(N), sizeof(T), R, 2);                \
    const int grid = grid_for(ceil_div(M, R), 2);                                                \
    BT_CHECK_LAUNCHED(launch_dependent(staged::rms_bwd_staged<T, V, R, ADD>, dim3(grid),          \
                                       dim3(staged::kThreads), smem, s, gp, xp, wp, rstd, dxp,   \
                                       dwp, wsp, M, static_cast<int>(N), ld_dy, ld_x, ld_dx, rp, \
                                       rr.ld_dres),                                              \
                      "rms_bwd_staged");                                                         \
    return BT_OK;                                                                                \
  }
    BT_BWDS(1, 4)
    BT_BWDS(2, 2)
    BT_BWDS(4, 1)
#undef BT_BWDS
  }
  if (vec_ok && pick_rows(nv, 4, &c)) {
    const int64_t rows_per_iter = static_cast<int64_t>(kThreads / c.lpr) * c.rpi;
    const size_t smem = static_cast<size_t>(N) * sizeof(float);
    // One wave exactly: the kernel walks its rows with a grid stride and ends with one set of
    // column-sum reductions per CTA, so the grid is what is resident at once (3 CTAs per SM at its
    // register count; 4 per SM meant a second wave at a third of the occupancy).
#define BT_BWD(L, V, R)                                                                         \
  if (c.lpr == L && c.vpt == V) {                                                               \
    static const int resident = resident_ctas(rms_bwd_rows<T, V, L, R, ADD>, kThreads, 4 * 1024);  \
    const int grid = grid_for(ceil_div(M, rows_per_iter), resident);                            \
    BT_CHECK_LAUNCHED(launch_dependent(rms_bwd_rows<T, V, L, R, ADD>, dim3(grid), dim3(kThreads),  \
                                       smem, s, gp, xp, wp, rstd, dxp, dwp, wsp, M,             \
                                       static_cast<int>(N), ld_dy, ld_x, ld_dx, rp, rr.ld_dres), \
                      "rms_bwd_rows");                                                          \
    return BT_OK;                                                                               \
  }
    BT_BWD(8, 1, 4)
    BT_BWD(16, 1, 4)
    BT_BWD(32, 1, 4)
    BT_BWD(32, 2, 2)
    BT_BWD(32, 4, 1)
#undef BT_BWD
  }
  rms_bwd_dx_generic<T><<<grid_for(M, 8), kThreads, 0, s>>>(gp, xp, wp, rstd, dxp, M, N, ld_dy,
                                                            ld_x, ld_dx, rp, rr.ld_dres);
  BT_CHECK_LAUNCH("rms_bwd_dx_generic");
  dim3 g(static_cast<unsigned>(ceil_div(N, 32)),
         static_cast<unsigned>(M < 8 * 64 ? 1 : (M / 8 < 64 ? M / 8 : 64)));
  rms_bwd_dw_generic<T><<<g, dim3(32, 8), 0, s>>>(gp, xp, rstd, dwp, wsp, M, static_cast<int>(N),
                                                  ld_dy, ld_x);
  BT_CHECK_LAUNCH("rms_bwd_dw_generic");
  return BT_OK;
}

template <bool ADD>
int fwd_any(int dtype, const void* x, const void* w, void* y, float* rstd, int64_t M, int64_t N,
            int64_t ld_x, int64_t ld_y, float eps, const Residual& rr, cudaStream_t s) {
  switch (dtype) {
    case BT_BF16: return fwd_t<__nv_bfloat16, ADD>(x, w, y, rstd, M, N, ld_x, ld_y, eps, rr, s);
    case BT_FP16: return fwd_t<__half, ADD>(x, w, y, rstd, M, N, ld_x, ld_y, eps, rr, s);
    case BT_FP32: return fwd_t<float, ADD>(x, w, y, rstd, M, N, ld_x, ld_y, eps, rr, s);
  }
  set_error("rmsnorm_fwd: unknown dtype %d", dtype);
  return BT_ERR_ARG;
}

template <bool ADD>
int bwd_any(int dtype, const void* dy, const void* x, const void* w, const float* rstd, void* dx,
            void* dw, void* ws, int64_t M, int64_t N, int64_t ld_dy, int64_t ld_x, int64_t ld_dx,
            const Residual& rr, cudaStream_t s) {
  switch (dtype) {
    case BT_BF16:
      return bwd_t<__nv_bfloat16, ADD>(dy, x, w, rstd, dx, dw, ws, M, N, ld_dy, ld_x, ld_dx, rr, s);
    case BT_FP16:
      return bwd_t<__half, ADD>(dy, x, w, rstd, dx, dw, ws, M, N, ld_dy, ld_x, ld_dx, rr, s);
    case BT_FP32:
      return bwd_t<float, ADD>(dy, x, w, rstd, dx, dw, ws, M, N, ld_dy, ld_x, ld_dx, rr, s);
  }
  set_error("rmsnorm_bwd: unknown dtype %d", dtype);
  return BT_ERR_ARG;
}

// dw of an empty batch: zero.  The scratch is all zeros by contract, so the finalize path
// of the generic dw kernel with an empty row range writes exactly that.
int bwd_empty(int dtype, void* dw, void* ws, int64_t N, cudaStream_t s) {
  dim3 g(static_cast<unsigned>(ceil_div(N, 32)), 1);
  float* wsp = static_cast<float*>(ws);
  const int n = static_cast<int>(N);
  switch (dtype) {
    case BT_BF16:
      rms_bwd_dw_generic<__nv_bfloat16><<<g, dim3(32, 8), 0, s>>>(
          nullptr, nullptr, nullptr, static_cast<__nv_bfloat16*>(dw), wsp, 0, n, 0, 0);
      break;
    case BT_FP16:
      rms_bwd_dw_generic<__half><<<g, dim3(32, 8), 0, s>>>(nullptr, nullptr, nullptr,
                                                          static_cast<__half*>(dw), wsp, 0, n, 0, 0);
      break;
    case BT_FP32:
      rms_bwd_dw_generic<float><<<g, dim3(32, 8), 0, s>>>(nullptr, nullptr, nullptr,
                                                         static_cast<float*>(dw), wsp, 0, n, 0, 0);
      break;
    default: set_error("rmsnorm_bwd: unknown dtype %d", dtype); return BT_ERR_ARG;
  }
  BT_CHECK_LAUNCH("rms_bwd_dw_generic(empty)");
  return BT_OK;
}

}  // namespace
}  // namespace bt

extern "C" int bt_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int64_t M,
                              int64_t N, int64_t ld_x, int64_t ld_y, float eps, int dtype,
                              void* stream) {
  using namespace bt;
  BT_CHECK_ARG(M >= 0 && N > 0 && N < (1ll << 31), "rmsnorm_fwd: bad shape M=%lld N=%lld",
               (long long)M, (long long)N);
  BT_CHECK_ARG(ld_x >= N && ld_y >= N, "rmsnorm_fwd: row stride smaller than N");
  if (M == 0) return BT_OK;
  BT_CHECK_ARG(x && w && y && rstd, "rmsnorm_fwd: null pointer");
  return fwd_any<false>(dtype, x, w, y, rstd, M, N, ld_x, ld_y, eps, Residual{},
                        static_cast<cudaStream_t>(stream));
}

extern "C" int bt_add_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* sum,
                                  void* y, float* rstd, int64_t M, int64_t N, int64_t ld_x,
                                  int64_t ld_residual, int64_t ld_sum, int64_t ld_y, float eps,
                                  int dtype, void* stream) {
  using namespace bt;
  BT_CHECK_ARG(M >= 0 && N > 0 && N < (1ll << 31), "add_rmsnorm_fwd: bad shape M=%lld N=%lld",
               (long long)M, (long long)N);
  BT_CHECK_ARG(ld_x >= N && ld_y >= N && ld_residual >= N && ld_sum >= N,
               "add_rmsnorm_fwd: row stride smaller than N");
  if (M == 0) return BT_OK;
  BT_CHECK_ARG(x && residual && w && sum && y && rstd, "add_rmsnorm_fwd: null pointer");
  BT_CHECK_ARG(sum != x && sum != residual && sum != y, "add_rmsnorm_fwd: sum must not alias");
  Residual rr;
  rr.res = residual;
  rr.sum = sum;
  rr.ld_res = ld_residual;
  rr.ld_sum = ld_sum;
  return fwd_any<true>(dtype, x, w, y, rstd, M, N, ld_x, ld_y, eps, rr,
                       static_cast<cudaStream_t>(stream));
}

extern "C" int64_t bt_rmsnorm_bwd_ws_bytes(int64_t N) {
  return (static_cast<int64_t>(bt::dw_copies(N)) * N + 1) * 4;
}

int bt_internal_set_wait_limit_tc(unsigned long long ns);  // tc_ops.cu

extern "C" int bt_set_wait_limit_ms(int64_t ms) {
  using namespace bt;
  BT_CHECK_ARG(ms >= 1 && ms <= 600000, "set_wait_limit_ms: the limit must be 1 ms .. 10 min");
  const unsigned long long ns = static_cast<unsigned long long>(ms) * 1000000ull;
  if (ptx::set_wait_limit_ns(ns) != cudaSuccess || bt_internal_set_wait_limit_tc(ns) != 0) {
    set_error("set_wait_limit_ms: writing the limit to the device failed");
    return BT_ERR_LAUNCH;
  }
  return BT_OK;
}

extern "C" int bt_device_wait_errors(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, bt::staged::g_wait_error, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(bt::staged::g_wait_error, &zero, sizeof(int));
  }
  return v;
}

extern "C" int bt_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd,
                              void* dx, void* dw, void* ws, int64_t M, int64_t N, int64_t ld_dy,
                              int64_t ld_x, int64_t ld_dx, int dtype, void* stream) {
  using namespace bt;
  BT_CHECK_ARG(M >= 0 && N > 0 && N < (1ll << 31), "rmsnorm_bwd: bad shape M=%lld N=%lld",
               (long long)M, (long long)N);
  BT_CHECK_ARG(ld_x >= N && ld_dy >= N && ld_dx >= N, "rmsnorm_bwd: row stride smaller than N");
  BT_CHECK_ARG(dw && ws, "rmsnorm_bwd: null dw / ws");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (M == 0) return bwd_empty(dtype, dw, ws, N, s);
  BT_CHECK_ARG(dy && x && w && rstd && dx, "rmsnorm_bwd: null pointer");
  return bwd_any<false>(dtype, dy, x, w, rstd, dx, dw, ws, M, N, ld_dy, ld_x, ld_dx, Residual{}, s);
}

extern "C" int bt_add_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd,
                                  const void* dresidual, void* dx, void* dw, void* ws, int64_t M,
                                  int64_t N, int64_t ld_dy, int64_t ld_x, int64_t ld_dresidual,
                                  int64_t ld_dx, int dtype, void* stream) {
  using namespace bt;
  BT_CHECK_ARG(M >= 0 && N > 0 && N < (1ll << 31), "add_rmsnorm_bwd: bad shape M=%lld N=%lld",
               (long long)M, (long long)N);
  BT_CHECK_ARG(ld_x >= N && ld_dy >= N && ld_dx >= N && ld_dresidual >= N,
               "add_rmsnorm_bwd: row stride smaller than N");
  BT_CHECK_ARG(dw && ws, "add_rmsnorm_bwd: null dw / ws");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (M == 0) return bwd_empty(dtype, dw, ws, N, s);
  BT_CHECK_ARG(dy && x && w && rstd && dx && dresidual, "add_rmsnorm_bwd: null pointer");
  BT_CHECK_ARG(dx != dresidual && dx != dy && dx != x, "add_rmsnorm_bwd: dx must not alias an input");
  Residual rr;
  rr.dres = dresidual;
  rr.ld_dres = ld_dresidual;
  return bwd_any<true>(dtype, dy, x, w, rstd, dx, dw, ws, M, N, ld_dy, ld_x, ld_dx, rr, s);
}

// ---------------------------------------------------------------------------
// bt_rmsnorm_bwd_noalloc: the same backward for callers that have no scratch
// buffer to hand over and no way to get one.
//
// Who that is: a host program that embeds this library behind an FFI and owns no
// device allocator of its own (it receives its tensors from a framework and may
// not call cudaMalloc behind that framework's back, because the framework has
// reserved the device memory for its own pool), and code on a latency-critical
// path where the implicit device-wide synchronisation of cudaMalloc / cudaFree is
// not acceptable.  For them the column-sum scratch lives in the library image
// itself, in the fixed-size device array below.  The price: every GPU that loads
// the library carries the array until the process exits, N is capped at
// BT_RMSNORM_NOALLOC_MAX_N, and all calls on one GPU share the one array.
namespace bt {
namespace {

constexpr int kNoAllocMaxN = BT_RMSNORM_NOALLOC_MAX_N;

// Column sums (fp32) followed by the arrival counter used by dw_finalize.
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocMaxN + 64];

// In host code `g_noalloc_scratch` is only a handle for the runtime, not an
// address a kernel may dereference: the device address has to be asked for, per
// device, with that device current.  Cached after the first successful query.
std::mutex g_noalloc_mu;
float* g_noalloc_ptr[64] = {nullptr};

int noalloc_scratch(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    set_error("rmsnorm_bwd_noalloc: cudaGetDevice failed: %s", cudaGetErrorString(e));
    return BT_ERR_LAUNCH;
  }
  std::lock_guard<std::mutex> lock(g_noalloc_mu);
  if (g_noalloc_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_error("rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev,
                cudaGetErrorString(e));
      return BT_ERR_LAUNCH;
    }
    g_noalloc_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_noalloc_ptr[dev];
  return BT_OK;
}

}  // namespace
}  // namespace bt

extern "C" int bt_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w,
                                      const float* rstd, void* dx, void* dw, int64_t M, int64_t N,
                                      int64_t ld_dy, int64_t ld_x, int64_t ld_dx, int dtype,
                                      void* stream) {
  using namespace bt;
  if (N > kNoAllocMaxN) {
    set_error("rmsnorm_bwd_noalloc: N = %lld exceeds the built-in scratch (max %d columns); "
              "use bt_rmsnorm_bwd with a caller-owned scratch buffer",
              (long long)N, kNoAllocMaxN);
    return BT_ERR_LIMIT;
  }
  BT_CHECK_ARG(N > 0, "rmsnorm_bwd_noalloc: N must be positive");
  float* scratch = nullptr;
  if (int rc = noalloc_scratch(&scratch)) return rc;
  // The array keeps whatever the previous call (or a call that was cut short) left in
  // it; the kernels need zeros in the N sums and in the counter.
  cudaError_t e = cudaMemsetAsync(scratch, 0, static_cast<size_t>(bt_rmsnorm_bwd_ws_bytes(N)),
                                  static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    set_error("rmsnorm_bwd_noalloc: clearing the scratch failed: %s", cudaGetErrorString(e));
    return BT_ERR_LAUNCH;
  }
  return bt_rmsnorm_bwd(dy, x, w, rstd, dx, dw, scratch, M, N, ld_dy, ld_x, ld_dx, dtype, stream);
}

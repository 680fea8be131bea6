// Per-head RMSNorm followed by rotate-half RoPE as ONE pass over a [B,T,H,D] tensor of heads
// (the q_norm / k_norm + apply_rotary_pos_emb sequence of Qwen3 attention), forward and
// backward.  Bandwidth-bound: each head row (D elements, 128 to 512 bytes) is read once and
// written once; unfused, the same row makes three round trips (norm, then RoPE in place).
//
// Layout: a group of LPR lanes owns one head row, one 16-byte vector per lane, so
// D = LPR * (elements per vector).  Lane l < LPR/2 holds a slice of the first half of the
// row, lane l + LPR/2 the matching slice of the second half: the rotation partner is one
// shuffle away, and both use the same slice of the cos/sin half row.  The row sum of
// squares (and the backward's dot product) is a shuffle reduction inside the group.  A
// 256-thread CTA works on (256 / LPR) * kRowsPerIter rows per iteration, all loads issued
// before the first use.
//
// Rounding points are those of the unfused pair: the normalised row is rounded to the
// storage type before it is rotated, and the backward rounds the un-rotated gradient before
// it enters the norm's backward - so results are bit-identical to bt_rmsnorm_* + bt_rope.
#include "bt_common.cuh"

namespace bt {
namespace {

constexpr int kThreads = 256;
constexpr int kRowsPerIter = 4;

struct HeadArgs {
  const void* x;     // [B,T,H,D] projection output (strides xs)
  const void* w;     // [D]
  const void* cos;   // [cos_bs, T, >= D/2]
  const void* sin;
  const void* dout;  // backward: gradient of the rotated output (strides gs)
  const float* rstd_in;
  void* out;         // forward: rotated output (strides os); backward: dx
  float* rstd_out;
  void* dw;
  float* ws;
  int64_t B, T, H;
  int D;
  int64_t xs[3], os[3], gs[3];  // element strides of (batch, position, head)
  int64_t cs[2];
  int cos_bs;
  float eps;
};

template <typename T>
__device__ __forceinline__ float round_to(float v) {
  return Cvt<T>::to_f(Cvt<T>::from_f(v));
}

template <typename T, int LPR>
__global__ void __launch_bounds__(kThreads, 4) headnorm_rope_fwd(const HeadArgs a) {
  constexpr int E = Cvt<T>::N;
  constexpr int kGroups = kThreads / LPR;
  constexpr int kHalf = LPR / 2;
  const int lane = threadIdx.x % LPR;
  const int group = threadIdx.x / LPR;
  const int j = lane % kHalf;
  const bool second = lane >= kHalf;
  const int64_t M = a.B * a.T * a.H;
  const float inv_n = 1.0f / static_cast<float>(a.D);
  const int64_t rows_per_iter = static_cast<int64_t>(kGroups) * kRowsPerIter;

  float wf[E];
  Cvt<T>::unpack(ld_global_v4(static_cast<const T*>(a.w) + lane * E), wf);

  for (int64_t base = static_cast<int64_t>(blockIdx.x) * rows_per_iter; base < M;
       base += static_cast<int64_t>(gridDim.x) * rows_per_iter) {
    uint4 xv[kRowsPerIter], cv[kRowsPerIter], sv[kRowsPerIter];
    T* outp[kRowsPerIter];
#pragma unroll
    for (int r = 0; r < kRowsPerIter; ++r) {
      const int64_t row = base + r * kGroups + group;
      outp[r] = nullptr;
      xv[r] = cv[r] = sv[r] = make_uint4(0, 0, 0, 0);
      if (row < M) {
        const int64_t h = row % a.H;
        const int64_t t = (row / a.H) % a.T;
        const int64_t b = row / (a.H * a.T);
        const int64_t cb = (a.cos_bs == 1) ? 0 : b;
        xv[r] = ld_stream_v4(static_cast<const T*>(a.x) + b * a.xs[0] + t * a.xs[1] + h * a.xs[2] +
                             lane * E);
        cv[r] = ld_global_v4(static_cast<const T*>(a.cos) + cb * a.cs[0] + t * a.cs[1] + j * E);
        sv[r] = ld_global_v4(static_cast<const T*>(a.sin) + cb * a.cs[0] + t * a.cs[1] + j * E);
        outp[r] = static_cast<T*>(a.out) + b * a.os[0] + t * a.os[1] + h * a.os[2] + lane * E;
      }
    }
#pragma unroll
    for (int r = 0; r < kRowsPerIter; ++r) {
      const int64_t row = base + r * kGroups + group;
      float f[E], c[E], s[E], o[E];
      Cvt<T>::unpack(xv[r], f);
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < E; ++e) ss = fmaf(f[e], f[e], ss);
      ss = group_sum<LPR>(ss);
      const float rs = rsqrtf(ss * inv_n + a.eps);
      Cvt<T>::unpack(cv[r], c);
      Cvt<T>::unpack(sv[r], s);
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const float y = round_to<T>(f[e] * rs * wf[e]);
        const float partner = __shfl_xor_sync(0xffffffffu, y, kHalf);
        // first half: y1*cos - y2*sin ; second half: y2*cos + y1*sin
        o[e] = second ? fmaf(partner, s[e], y * c[e]) : fmaf(-partner, s[e], y * c[e]);
      }
      if (outp[r] != nullptr) {
        if (lane == 0) a.rstd_out[row] = rs;
        st_global_v4(outp[r], Cvt<T>::pack(o));
      }
    }
  }
}

// dx, dw of the fused pair.  ws: dw_copies(D) x D fp32 column sums + arrival counter, zero
// on entry, left zero on exit (the contract of the RMSNorm backward).
template <typename T, int LPR>
__global__ void __launch_bounds__(kThreads, 3) headnorm_rope_bwd(const HeadArgs a) {
  constexpr int E = Cvt<T>::N;
  constexpr int kGroups = kThreads / LPR;
  constexpr int kHalf = LPR / 2;
  __shared__ float s_dw[LPR * E];
  const int lane = threadIdx.x % LPR;
  const int group = threadIdx.x / LPR;
  const int j = lane % kHalf;
  const bool second = lane >= kHalf;
  const int N = a.D;
  const int64_t M = a.B * a.T * a.H;
  const float inv_n = 1.0f / static_cast<float>(N);
  const int64_t rows_per_iter = static_cast<int64_t>(kGroups) * kRowsPerIter;

  for (int c = threadIdx.x; c < N; c += kThreads) s_dw[c] = 0.f;

  float wf[E], acc[E];
  Cvt<T>::unpack(ld_global_v4(static_cast<const T*>(a.w) + lane * E), wf);
#pragma unroll
  for (int e = 0; e < E; ++e) acc[e] = 0.f;

  for (int64_t base = static_cast<int64_t>(blockIdx.x) * rows_per_iter; base < M;
       base += static_cast<int64_t>(gridDim.x) * rows_per_iter) {
    uint4 xv[kRowsPerIter], gv[kRowsPerIter], cv[kRowsPerIter], sv[kRowsPerIter];
    float rs[kRowsPerIter];
    T* outp[kRowsPerIter];
#pragma unroll
    for (int r = 0; r < kRowsPerIter; ++r) {
      const int64_t row = base + r * kGroups + group;
      outp[r] = nullptr;
      rs[r] = 0.f;
      xv[r] = gv[r] = cv[r] = sv[r] = make_uint4(0, 0, 0, 0);
      if (row < M) {
        const int64_t h = row % a.H;
        const int64_t t = (row / a.H) % a.T;
        const int64_t b = row / (a.H * a.T);
        const int64_t cb = (a.cos_bs == 1) ? 0 : b;
        rs[r] = a.rstd_in[row];
        xv[r] = ld_stream_v4(static_cast<const T*>(a.x) + b * a.xs[0] + t * a.xs[1] + h * a.xs[2] +
                             lane * E);
        gv[r] = ld_stream_v4(static_cast<const T*>(a.dout) + b * a.gs[0] + t * a.gs[1] +
                             h * a.gs[2] + lane * E);
        cv[r] = ld_global_v4(static_cast<const T*>(a.cos) + cb * a.cs[0] + t * a.cs[1] + j * E);
        sv[r] = ld_global_v4(static_cast<const T*>(a.sin) + cb * a.cs[0] + t * a.cs[1] + j * E);
        outp[r] = static_cast<T*>(a.out) + b * a.os[0] + t * a.os[1] + h * a.os[2] + lane * E;
      }
    }
#pragma unroll
    for (int r = 0; r < kRowsPerIter; ++r) {
      float xf[E], gf[E], c[E], s[E], dy[E], o[E];
      Cvt<T>::unpack(xv[r], xf);
      Cvt<T>::unpack(gv[r], gf);
      Cvt<T>::unpack(cv[r], c);
      Cvt<T>::unpack(sv[r], s);
      float dot = 0.f;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const float partner = __shfl_xor_sync(0xffffffffu, gf[e], kHalf);
        // inverse rotation: d1*cos + d2*sin ; d2*cos - d1*sin
        dy[e] = round_to<T>(second ? fmaf(-partner, s[e], gf[e] * c[e])
                                   : fmaf(partner, s[e], gf[e] * c[e]));
        const float xh = xf[e] * rs[r];
        dot = fmaf(xh, dy[e] * wf[e], dot);
        acc[e] = fmaf(dy[e], xh, acc[e]);
      }
      dot = group_sum<LPR>(dot) * inv_n;
      if (outp[r] != nullptr) {
#pragma unroll
        for (int e = 0; e < E; ++e) o[e] = fmaf(-(xf[e] * rs[r]), dot, dy[e] * wf[e]) * rs[r];
        st_global_v4(outp[r], Cvt<T>::pack(o));
      }
    }
  }

  __syncthreads();  // s_dw zeroed
  // Row groups that share a warp hold the same columns: fold them together first.
#pragma unroll
  for (int o = LPR; o < 32; o <<= 1) {
#pragma unroll
    for (int e = 0; e < E; ++e) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], o);
  }
  // element-major in shared memory (index e * LPR + lane): lanes of one instruction hit
  // different banks
  if ((threadIdx.x & 31) < LPR) {
#pragma unroll
    for (int e = 0; e < E; ++e) atomicAdd(&s_dw[e * LPR + lane], acc[e]);
  }
  __syncthreads();
  float* my_ws = a.ws + static_cast<int64_t>(blockIdx.x % dw_copies(N)) * N;
  for (int c = threadIdx.x; c < N; c += kThreads) atomicAdd(my_ws + c, s_dw[(c % E) * LPR + c / E]);
  dw_finalize<T>(a.ws, static_cast<T*>(a.dw), N, gridDim.x, threadIdx.x, kThreads);
}

bool mult_of(const int64_t* s, int n, int e) {
  for (int i = 0; i < n; ++i)
    if (s[i] % e != 0) return false;
  return true;
}

template <typename T, bool BWD>
int launch_t(const HeadArgs& a, cudaStream_t s) {
  constexpr int E = Cvt<T>::N;
  const int lpr = a.D / E;
  bool ok = a.D % E == 0 && (lpr == 8 || lpr == 16 || lpr == 32) && aligned16(a.x) &&
            aligned16(a.w) && aligned16(a.cos) && aligned16(a.sin) && aligned16(a.out) &&
            mult_of(a.xs, 3, E) && mult_of(a.os, 3, E) && mult_of(a.cs, 2, E);
  if (BWD) ok = ok && aligned16(a.dout) && mult_of(a.gs, 3, E);
  if (!ok) {
    set_error("headnorm_rope: head_dim %d with this element size / alignment is not supported "
              "(head rows of 128, 256 or 512 bytes, 16-byte aligned strides); run the norm and "
              "the rotation as separate calls",
              a.D);
    return BT_ERR_ARG;
  }
  const int64_t M = a.B * a.T * a.H;
  const int64_t rows_per_iter = static_cast<int64_t>(kThreads / lpr) * kRowsPerIter;
  const int64_t blocks = ceil_div(M, rows_per_iter);
  const int64_t cap = static_cast<int64_t>(sm_count()) * (BWD ? 4 : 32);
  const unsigned grid = static_cast<unsigned>(blocks < cap ? blocks : cap);
#define BT_HEAD(L)                                                         \
  if (lpr == L) {                                                          \
    if (BWD)                                                               \
      headnorm_rope_bwd<T, L><<<grid, kThreads, 0, s>>>(a);                \
    else                                                                   \
      headnorm_rope_fwd<T, L><<<grid, kThreads, 0, s>>>(a);                \
  }
  BT_HEAD(8)
  BT_HEAD(16)
  BT_HEAD(32)
#undef BT_HEAD
  BT_CHECK_LAUNCH(BWD ? "headnorm_rope_bwd" : "headnorm_rope_fwd");
  return BT_OK;
}

template <bool BWD>
int launch_any(int dtype, const HeadArgs& a, cudaStream_t s) {
  switch (dtype) {
    case BT_BF16: return launch_t<__nv_bfloat16, BWD>(a, s);
    case BT_FP16: return launch_t<__half, BWD>(a, s);
    case BT_FP32: return launch_t<float, BWD>(a, s);
  }
  set_error("headnorm_rope: unknown dtype %d", dtype);
  return BT_ERR_ARG;
}

int fill_common(HeadArgs* a, const char* what, int64_t B, int64_t T, int64_t H, int64_t D,
                const int64_t cos_strides[2], int64_t cos_bs) {
  BT_CHECK_ARG(B >= 0 && T >= 0 && H >= 0, "%s: negative size", what);
  BT_CHECK_ARG(D > 0 && D % 2 == 0 && D <= 4096, "%s: head_dim %lld must be even and <= 4096", what,
               (long long)D);
  BT_CHECK_ARG(cos_bs == 1 || cos_bs == B, "%s: cos batch %lld is neither 1 nor B=%lld", what,
               (long long)cos_bs, (long long)B);
  a->B = B;
  a->T = T;
  a->H = H;
  a->D = static_cast<int>(D);
  a->cs[0] = cos_strides[0];
  a->cs[1] = cos_strides[1];
  a->cos_bs = static_cast<int>(cos_bs);
  return BT_OK;
}

}  // namespace
}  // namespace bt

extern "C" int bt_headnorm_rope_fwd(const void* x, const void* w, const void* cos, const void* sin,
                                    void* out, float* rstd, int64_t B, int64_t T, int64_t H,
                                    int64_t D, const int64_t x_strides[3],
                                    const int64_t out_strides[3], const int64_t cos_strides[2],
                                    int64_t cos_bs, float eps, int dtype, void* stream) {
  using namespace bt;
  HeadArgs a{};
  if (int rc = fill_common(&a, "headnorm_rope_fwd", B, T, H, D, cos_strides, cos_bs)) return rc;
  if (B == 0 || T == 0 || H == 0) return BT_OK;
  BT_CHECK_ARG(x && w && cos && sin && out && rstd, "headnorm_rope_fwd: null pointer");
  a.x = x;
  a.w = w;
  a.cos = cos;
  a.sin = sin;
  a.out = out;
  a.rstd_out = rstd;
  a.eps = eps;
  for (int i = 0; i < 3; ++i) {
    a.xs[i] = x_strides[i];
    a.os[i] = out_strides[i];
  }
  return launch_any<false>(dtype, a, static_cast<cudaStream_t>(stream));
}

extern "C" int bt_headnorm_rope_bwd(const void* dout, const void* x, const void* w,
                                    const float* rstd, const void* cos, const void* sin, void* dx,
                                    void* dw, void* ws, int64_t B, int64_t T, int64_t H, int64_t D,
                                    const int64_t dout_strides[3], const int64_t x_strides[3],
                                    const int64_t dx_strides[3], const int64_t cos_strides[2],
                                    int64_t cos_bs, int dtype, void* stream) {
  using namespace bt;
  HeadArgs a{};
  if (int rc = fill_common(&a, "headnorm_rope_bwd", B, T, H, D, cos_strides, cos_bs)) return rc;
  BT_CHECK_ARG(B > 0 && T > 0 && H > 0, "headnorm_rope_bwd: empty input");
  BT_CHECK_ARG(dout && x && w && rstd && cos && sin && dx && dw && ws,
               "headnorm_rope_bwd: null pointer");
  a.dout = dout;
  a.x = x;
  a.w = w;
  a.rstd_in = rstd;
  a.cos = cos;
  a.sin = sin;
  a.out = dx;
  a.dw = dw;
  a.ws = static_cast<float*>(ws);
  for (int i = 0; i < 3; ++i) {
    a.gs[i] = dout_strides[i];
    a.xs[i] = x_strides[i];
    a.os[i] = dx_strides[i];
  }
  return launch_any<true>(dtype, a, static_cast<cudaStream_t>(stream));
}

// Per-head RMSNorm followed by rotate-half RoPE as ONE pass over a [B,T,H,D] tensor of heads
// (the q_norm / k_norm + apply_rotary_pos_emb sequence of Qwen3 attention), forward and
// backward.  Bandwidth-bound: each head row (D elements, 128 to 512 bytes) is read once and
// written once; unfused, the same row makes three round trips (norm, then RoPE in place).
//
// Layout: a group of LPR lanes owns one head row; a lane holds one 16-byte slice of the first
// half of the row and the matching slice of the second half (D = 2 * LPR * elements per
// vector), so the rotation needs no exchange between lanes and both slices use the same
// 16 bytes of the cos/sin half row.  The row sum of squares (and the backward's dot product)
// is a shuffle reduction inside the group.  A 256-thread CTA works on 256 / LPR items per
// iteration, an item being one token's block of 4 (backward: 2) consecutive heads, with all
// of an item's loads issued before the first use.
//
// Rounding points are those of the unfused pair: the normalised row is rounded to the
// storage type before it is rotated, and the backward rounds the un-rotated gradient before
// it enters the norm's backward - so results are bit-identical to bt_rmsnorm_* + bt_rope.
#include "bt_common.cuh"

namespace bt {
namespace {

constexpr int kThreads = 256;

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

// Work item = (token, block of HPI consecutive heads): the heads of one token share the
// token's cos/sin slice, and in [B,T,H,D] storage they are adjacent in memory.
struct Item {
  bool valid;
  int64_t x_off, g_off, o_off, c_off, row0;  // element offsets of head h0; rstd index of head h0
  int h0;
};

template <int HPI>
__device__ __forceinline__ Item locate(const HeadArgs& a, uint32_t item, uint32_t items,
                                       uint32_t hblocks) {
  Item it;
  it.valid = item < items;
  const uint32_t bt = it.valid ? item / hblocks : 0u;
  const uint32_t hb = it.valid ? item - bt * hblocks : 0u;
  const uint32_t b = bt / static_cast<uint32_t>(a.T);
  const uint32_t t = bt - b * static_cast<uint32_t>(a.T);
  it.h0 = static_cast<int>(hb) * HPI;
  it.x_off = b * a.xs[0] + t * a.xs[1] + it.h0 * a.xs[2];
  it.g_off = b * a.gs[0] + t * a.gs[1] + it.h0 * a.gs[2];
  it.o_off = b * a.os[0] + t * a.os[1] + it.h0 * a.os[2];
  it.c_off = (a.cos_bs == 1 ? 0 : b * a.cs[0]) + t * a.cs[1];
  it.row0 = static_cast<int64_t>(bt) * a.H + it.h0;
  return it;
}

// Row sums are formed in the order the stand-alone RMSNorm kernels use for a row of this
// width (a chain per 16-byte slice, first-half slice + matching second-half slice, then a
// butterfly over the slices), which keeps rstd and the backward's dot product bit-identical.
template <typename T, int LPR, int HPI, int MINB>
__global__ void __launch_bounds__(kThreads, MINB) headnorm_rope_fwd(const HeadArgs a) {
  constexpr int E = Cvt<T>::N;
  constexpr int kGroups = kThreads / LPR;
  const int lane = threadIdx.x % LPR;
  const int group = threadIdx.x / LPR;
  const int half = a.D / 2;
  const int H = static_cast<int>(a.H);
  const uint32_t hblocks = static_cast<uint32_t>((H + HPI - 1) / HPI);
  const uint32_t items = static_cast<uint32_t>(a.B * a.T) * hblocks;
  const float inv_n = 1.0f / static_cast<float>(a.D);

  float w1[E], w2[E];
  Cvt<T>::unpack(ld_global_v4(static_cast<const T*>(a.w) + lane * E), w1);
  Cvt<T>::unpack(ld_global_v4(static_cast<const T*>(a.w) + half + lane * E), w2);

  for (uint32_t base = blockIdx.x * kGroups; base < items; base += gridDim.x * kGroups) {
    const Item it = locate<HPI>(a, base + group, items, hblocks);
    uint4 x1[HPI], x2[HPI];
    uint4 cv = make_uint4(0, 0, 0, 0), sv = make_uint4(0, 0, 0, 0);
    if (it.valid) {
      cv = ld_global_v4(static_cast<const T*>(a.cos) + it.c_off + lane * E);
      sv = ld_global_v4(static_cast<const T*>(a.sin) + it.c_off + lane * E);
    }
#pragma unroll
    for (int u = 0; u < HPI; ++u) {
      const bool ok = it.valid && it.h0 + u < H;
      const T* xp = static_cast<const T*>(a.x) + it.x_off + u * a.xs[2] + lane * E;
      x1[u] = ok ? ld_stream_v4(xp) : make_uint4(0, 0, 0, 0);
      x2[u] = ok ? ld_stream_v4(xp + half) : make_uint4(0, 0, 0, 0);
    }
    float c[E], s[E];
    Cvt<T>::unpack(cv, c);
    Cvt<T>::unpack(sv, s);
#pragma unroll
    for (int u = 0; u < HPI; ++u) {
      float f1[E], f2[E], o1[E], o2[E];
      Cvt<T>::unpack(x1[u], f1);
      Cvt<T>::unpack(x2[u], f2);
      float p1 = 0.f, p2 = 0.f;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        p1 = fmaf(f1[e], f1[e], p1);
        p2 = fmaf(f2[e], f2[e], p2);
      }
      const float ss = group_sum<LPR>(p1 + p2);
      const float rs = rsqrtf(ss * inv_n + a.eps);
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const float y1 = round_to<T>(f1[e] * rs * w1[e]);
        const float y2 = round_to<T>(f2[e] * rs * w2[e]);
        o1[e] = fmaf(-y2, s[e], y1 * c[e]);  // y1*cos - y2*sin
        o2[e] = fmaf(y1, s[e], y2 * c[e]);   // y2*cos + y1*sin
      }
      if (it.valid && it.h0 + u < H) {
        if (lane == 0) a.rstd_out[it.row0 + u] = rs;
        T* op = static_cast<T*>(a.out) + it.o_off + u * a.os[2] + lane * E;
        st_global_v4(op, Cvt<T>::pack(o1));
        st_global_v4(op + half, Cvt<T>::pack(o2));
      }
    }
  }
}

// dx, dw of the fused pair.  ws: dw_copies(D) x D fp32 column sums + arrival counter, zero
// on entry, left zero on exit (the contract of the RMSNorm backward).
template <typename T, int LPR, int HPI, int MINB>
__global__ void __launch_bounds__(kThreads, MINB) headnorm_rope_bwd(const HeadArgs a) {
  constexpr int E = Cvt<T>::N;
  constexpr int kGroups = kThreads / LPR;
  __shared__ float s_dw[2 * LPR * E];
  const int lane = threadIdx.x % LPR;
  const int group = threadIdx.x / LPR;
  const int N = a.D;
  const int half = N / 2;
  const int H = static_cast<int>(a.H);
  const uint32_t hblocks = static_cast<uint32_t>((H + HPI - 1) / HPI);
  const uint32_t items = static_cast<uint32_t>(a.B * a.T) * hblocks;
  const float inv_n = 1.0f / static_cast<float>(N);

  for (int c = threadIdx.x; c < N; c += kThreads) s_dw[c] = 0.f;

  float w1[E], w2[E], acc1[E], acc2[E];
  Cvt<T>::unpack(ld_global_v4(static_cast<const T*>(a.w) + lane * E), w1);
  Cvt<T>::unpack(ld_global_v4(static_cast<const T*>(a.w) + half + lane * E), w2);
#pragma unroll
  for (int e = 0; e < E; ++e) acc1[e] = acc2[e] = 0.f;

  for (uint32_t base = blockIdx.x * kGroups; base < items; base += gridDim.x * kGroups) {
    const Item it = locate<HPI>(a, base + group, items, hblocks);
    uint4 x1[HPI], x2[HPI], g1[HPI], g2[HPI];
    float rs[HPI];
    uint4 cv = make_uint4(0, 0, 0, 0), sv = make_uint4(0, 0, 0, 0);
    if (it.valid) {
      cv = ld_global_v4(static_cast<const T*>(a.cos) + it.c_off + lane * E);
      sv = ld_global_v4(static_cast<const T*>(a.sin) + it.c_off + lane * E);
    }
#pragma unroll
    for (int u = 0; u < HPI; ++u) {
      const bool ok = it.valid && it.h0 + u < H;
      const T* xp = static_cast<const T*>(a.x) + it.x_off + u * a.xs[2] + lane * E;
      const T* gp = static_cast<const T*>(a.dout) + it.g_off + u * a.gs[2] + lane * E;
      rs[u] = ok ? a.rstd_in[it.row0 + u] : 0.f;
      x1[u] = ok ? ld_stream_v4(xp) : make_uint4(0, 0, 0, 0);
      x2[u] = ok ? ld_stream_v4(xp + half) : make_uint4(0, 0, 0, 0);
      g1[u] = ok ? ld_stream_v4(gp) : make_uint4(0, 0, 0, 0);
      g2[u] = ok ? ld_stream_v4(gp + half) : make_uint4(0, 0, 0, 0);
    }
    float c[E], s[E];
    Cvt<T>::unpack(cv, c);
    Cvt<T>::unpack(sv, s);
#pragma unroll
    for (int u = 0; u < HPI; ++u) {
      float xa[E], xb[E], ga[E], gb[E], d1[E], d2[E];
      Cvt<T>::unpack(x1[u], xa);
      Cvt<T>::unpack(x2[u], xb);
      Cvt<T>::unpack(g1[u], ga);
      Cvt<T>::unpack(g2[u], gb);
      float p1 = 0.f, p2 = 0.f;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        // inverse rotation: d1*cos + d2*sin ; d2*cos - d1*sin
        d1[e] = round_to<T>(fmaf(gb[e], s[e], ga[e] * c[e]));
        d2[e] = round_to<T>(fmaf(-ga[e], s[e], gb[e] * c[e]));
        const float h1 = xa[e] * rs[u], h2 = xb[e] * rs[u];
        p1 = fmaf(h1, d1[e] * w1[e], p1);
        p2 = fmaf(h2, d2[e] * w2[e], p2);
        acc1[e] = fmaf(d1[e], h1, acc1[e]);
        acc2[e] = fmaf(d2[e], h2, acc2[e]);
      }
      const float dot = group_sum<LPR>(p1 + p2) * inv_n;
      if (it.valid && it.h0 + u < H) {
        float o1[E], o2[E];
#pragma unroll
        for (int e = 0; e < E; ++e) {
          o1[e] = fmaf(-(xa[e] * rs[u]), dot, d1[e] * w1[e]) * rs[u];
          o2[e] = fmaf(-(xb[e] * rs[u]), dot, d2[e] * w2[e]) * rs[u];
        }
        T* op = static_cast<T*>(a.out) + it.o_off + u * a.os[2] + lane * E;
        st_global_v4(op, Cvt<T>::pack(o1));
        st_global_v4(op + half, Cvt<T>::pack(o2));
      }
    }
  }

  __syncthreads();  // s_dw zeroed
  // Row groups that share a warp hold the same columns: fold them together first.
#pragma unroll
  for (int o = LPR; o < 32; o <<= 1) {
#pragma unroll
    for (int e = 0; e < E; ++e) {
      acc1[e] += __shfl_xor_sync(0xffffffffu, acc1[e], o);
      acc2[e] += __shfl_xor_sync(0xffffffffu, acc2[e], o);
    }
  }
  // element-major in shared memory (index (2e + which half) * LPR + lane): lanes of one
  // instruction hit different banks
  if ((threadIdx.x & 31) < LPR) {
#pragma unroll
    for (int e = 0; e < E; ++e) {
      atomicAdd(&s_dw[(2 * e) * LPR + lane], acc1[e]);
      atomicAdd(&s_dw[(2 * e + 1) * LPR + lane], acc2[e]);
    }
  }
  __syncthreads();
  float* my_ws = a.ws + static_cast<int64_t>(blockIdx.x % dw_copies(N)) * N;
  for (int c = threadIdx.x; c < N; c += kThreads) {
    const int hsel = c >= half ? 1 : 0;
    const int cc = c - hsel * half;  // column inside its half: slice cc / E, element cc % E
    atomicAdd(my_ws + c, s_dw[(2 * (cc % E) + hsel) * LPR + cc / E]);
  }
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
  const int lpr = a.D / (2 * E);  // lanes per head row: each holds one slice of either half
  bool ok = a.D % (2 * E) == 0 && (lpr == 4 || lpr == 8 || lpr == 16) && aligned16(a.x) &&
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
  constexpr int kHpi = BWD ? 2 : 4;  // heads per work item: 16-byte loads in flight per lane = 2 (4) * kHpi
  const int64_t items = a.B * a.T * ceil_div(a.H, kHpi);
  if (items >= (1ll << 31) || a.B * a.T * a.H >= (1ll << 31)) {
    set_error("headnorm_rope: %lld head rows exceed the 32-bit work index", (long long)(a.B * a.T * a.H));
    return BT_ERR_ARG;
  }
  const int64_t blocks = ceil_div(items, kThreads / lpr);
  const int64_t cap = static_cast<int64_t>(sm_count()) * (BWD ? 2 : 8);
  const unsigned grid = static_cast<unsigned>(blocks < cap ? blocks : cap);
#define BT_HEAD(L)                                                         \
  if (lpr == L) {                                                          \
    if (BWD)                                                               \
      headnorm_rope_bwd<T, L, kHpi, 2><<<grid, kThreads, 0, s>>>(a);       \
    else                                                                   \
      headnorm_rope_fwd<T, L, kHpi, 3><<<grid, kThreads, 0, s>>>(a);       \
  }
  BT_HEAD(4)
  BT_HEAD(8)
  BT_HEAD(16)
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

// Per-head RMSNorm followed by rotate-half RoPE as ONE pass over the q and k tensors of heads,
// each [B,T,H,D] (the q_norm / k_norm + apply_rotary_pos_emb sequence of Qwen3 attention),
// forward and backward, one launch for both tensors.  Bandwidth-bound: each head row (D elements, 128 to 512 bytes) is read once and
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

// One launch serves two tensors of heads (q and k): CTAs [0, split) work on p[0], the rest
// on p[1], each side with its own weight, rstd, dw and scratch.
struct HeadPair {
  HeadArgs p[2];
  unsigned split;
};

// Rounds a 16-byte vector's worth of fp32 values to the storage type and back (paired
// conversions: half the instructions of rounding element by element).
template <typename T>
__device__ __forceinline__ void round_vec(float (&v)[Cvt<T>::N]) {
  if constexpr (sizeof(T) < 4) {
    const uint4 packed = Cvt<T>::pack(v);
    Cvt<T>::unpack(packed, v);
  }
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
__global__ void __launch_bounds__(kThreads, MINB)
headnorm_rope_fwd(const __grid_constant__ HeadPair pp) {
  constexpr int E = Cvt<T>::N;
  constexpr int kGroups = kThreads / LPR;
  grid_dependency_wait();
  const bool side = blockIdx.x >= pp.split;
  const HeadArgs& a = pp.p[side ? 1 : 0];
  const unsigned bid = side ? blockIdx.x - pp.split : blockIdx.x;
  const unsigned nblk = side ? gridDim.x - pp.split : pp.split;
  const int lane = threadIdx.x % LPR;
  const int group = threadIdx.x / LPR;
  const int half = a.D / 2;
  const int H = static_cast<int>(a.H);
  const uint32_t hblocks = static_cast<uint32_t>((H + HPI - 1) / HPI);
  const uint32_t items = static_cast<uint32_t>(a.B * a.T) * hblocks;
  const float inv_n = 1.0f / static_cast<float>(a.D);

  // Elementwise arithmetic runs on packed fp32 pairs (same results per element, half the issue
  // slots); the row sums keep their scalar chains, whose order is part of the bit-identity with
  // the stand-alone kernels.
  constexpr int P = E / 2;
  f32x2 w1[P], w2[P];
  unpack_pairs<T>(ld_global_v4(static_cast<const T*>(a.w) + lane * E), w1);
  unpack_pairs<T>(ld_global_v4(static_cast<const T*>(a.w) + half + lane * E), w2);

  for (uint32_t base = bid * kGroups; base < items; base += nblk * kGroups) {
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
    f32x2 c[P], s[P];
    unpack_pairs<T>(cv, c);
    unpack_pairs<T>(sv, s);
#pragma unroll
    for (int u = 0; u < HPI; ++u) {
      f32x2 y1[P], y2[P], o1[P], o2[P];
      unpack_pairs<T>(x1[u], y1);
      unpack_pairs<T>(x2[u], y2);
      float p1 = 0.f, p2 = 0.f;
#pragma unroll
      for (int e = 0; e < P; ++e) {  // element order 0, 1, 2, ... within each slice
        p1 = fmaf(lo_of(y1[e]), lo_of(y1[e]), p1);
        p2 = fmaf(lo_of(y2[e]), lo_of(y2[e]), p2);
        p1 = fmaf(hi_of(y1[e]), hi_of(y1[e]), p1);
        p2 = fmaf(hi_of(y2[e]), hi_of(y2[e]), p2);
      }
      const float ss = group_sum<LPR>(p1 + p2);
      const float rs = rsqrtf(ss * inv_n + a.eps);
      const f32x2 rs2 = pair(rs, rs);
#pragma unroll
      for (int e = 0; e < P; ++e) {
        y1[e] = mul2(mul2(y1[e], rs2), w1[e]);
        y2[e] = mul2(mul2(y2[e], rs2), w2[e]);
      }
      if constexpr (sizeof(T) < 4) {
        // the normalised row as the stand-alone norm kernel would have stored it
        unpack_pairs<T>(pack_pairs<T>(y1), y1);
        unpack_pairs<T>(pack_pairs<T>(y2), y2);
      }
#pragma unroll
      for (int e = 0; e < P; ++e) {
        o1[e] = fma2(neg2(y2[e]), s[e], mul2(y1[e], c[e]));  // y1*cos - y2*sin
        o2[e] = fma2(y1[e], s[e], mul2(y2[e], c[e]));   // y2*cos + y1*sin
      }
      if (it.valid && it.h0 + u < H) {
        if (lane == 0) a.rstd_out[it.row0 + u] = rs;
        T* op = static_cast<T*>(a.out) + it.o_off + u * a.os[2] + lane * E;
        st_global_v4(op, pack_pairs<T>(o1));
        st_global_v4(op + half, pack_pairs<T>(o2));
      }
    }
  }
}

// dx, dw of the fused pair.  ws: dw_copies(D) x D fp32 column sums + arrival counter, zero
// on entry, left zero on exit (the contract of the RMSNorm backward).
template <typename T, int LPR, int HPI, int MINB>
__global__ void __launch_bounds__(kThreads, MINB)
headnorm_rope_bwd(const __grid_constant__ HeadPair pp) {
  constexpr int E = Cvt<T>::N;
  constexpr int kGroups = kThreads / LPR;
  const bool side = blockIdx.x >= pp.split;
  const HeadArgs& a = pp.p[side ? 1 : 0];
  const unsigned bid = side ? blockIdx.x - pp.split : blockIdx.x;
  const unsigned nblk = side ? gridDim.x - pp.split : pp.split;
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
  grid_dependency_wait();

  // Elementwise arithmetic on packed fp32 pairs; the dot product keeps its scalar chains (their
  // order is part of the bit-identity with the stand-alone kernels).
  constexpr int P = E / 2;
  f32x2 w1[P], w2[P], acc1[P], acc2[P];
  unpack_pairs<T>(ld_global_v4(static_cast<const T*>(a.w) + lane * E), w1);
  unpack_pairs<T>(ld_global_v4(static_cast<const T*>(a.w) + half + lane * E), w2);
#pragma unroll
  for (int e = 0; e < P; ++e) acc1[e] = acc2[e] = pair(0.f, 0.f);

  for (uint32_t base = bid * kGroups; base < items; base += nblk * kGroups) {
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
    f32x2 c[P], s[P];
    unpack_pairs<T>(cv, c);
    unpack_pairs<T>(sv, s);
#pragma unroll
    for (int u = 0; u < HPI; ++u) {
      f32x2 h1[P], h2[P], d1[P], d2[P];
      {
        f32x2 ga[P], gb[P];
        unpack_pairs<T>(g1[u], ga);
        unpack_pairs<T>(g2[u], gb);
#pragma unroll
        for (int e = 0; e < P; ++e) {
          // inverse rotation: d1*cos + d2*sin ; d2*cos - d1*sin
          d1[e] = fma2(gb[e], s[e], mul2(ga[e], c[e]));
          d2[e] = fma2(neg2(ga[e]), s[e], mul2(gb[e], c[e]));
        }
      }
      if constexpr (sizeof(T) < 4) {
        // the un-rotated gradient as the stand-alone RoPE backward would have stored it
        unpack_pairs<T>(pack_pairs<T>(d1), d1);
        unpack_pairs<T>(pack_pairs<T>(d2), d2);
      }
      const f32x2 rs2 = pair(rs[u], rs[u]);
      unpack_pairs<T>(x1[u], h1);
      unpack_pairs<T>(x2[u], h2);
      float p1 = 0.f, p2 = 0.f;
#pragma unroll
      for (int e = 0; e < P; ++e) {
        h1[e] = mul2(h1[e], rs2);  // x * rstd
        h2[e] = mul2(h2[e], rs2);
        const f32x2 t1 = mul2(d1[e], w1[e]), t2 = mul2(d2[e], w2[e]);
        p1 = fmaf(lo_of(h1[e]), lo_of(t1), p1);  // element order 0, 1, 2, ... within each slice
        p2 = fmaf(lo_of(h2[e]), lo_of(t2), p2);
        p1 = fmaf(hi_of(h1[e]), hi_of(t1), p1);
        p2 = fmaf(hi_of(h2[e]), hi_of(t2), p2);
        acc1[e] = fma2(d1[e], h1[e], acc1[e]);
        acc2[e] = fma2(d2[e], h2[e], acc2[e]);
      }
      const float dot = group_sum<LPR>(p1 + p2) * inv_n;
      if (it.valid && it.h0 + u < H) {
        const f32x2 ndot = pair(-dot, -dot);
        f32x2 o1[P], o2[P];
#pragma unroll
        for (int e = 0; e < P; ++e) {
          // fmaf(-(x*rs), dot, d*w) * rs
          o1[e] = mul2(fma2(h1[e], ndot, mul2(d1[e], w1[e])), rs2);
          o2[e] = mul2(fma2(h2[e], ndot, mul2(d2[e], w2[e])), rs2);
        }
        T* op = static_cast<T*>(a.out) + it.o_off + u * a.os[2] + lane * E;
        st_global_v4(op, pack_pairs<T>(o1));
        st_global_v4(op + half, pack_pairs<T>(o2));
      }
    }
  }

  __syncthreads();  // s_dw zeroed
  // Row groups that share a warp hold the same columns: fold them together first.
  float a1[E], a2[E];
#pragma unroll
  for (int e = 0; e < P; ++e) {
    a1[2 * e] = lo_of(acc1[e]);
    a1[2 * e + 1] = hi_of(acc1[e]);
    a2[2 * e] = lo_of(acc2[e]);
    a2[2 * e + 1] = hi_of(acc2[e]);
  }
#pragma unroll
  for (int o = LPR; o < 32; o <<= 1) {
#pragma unroll
    for (int e = 0; e < E; ++e) {
      a1[e] += __shfl_xor_sync(0xffffffffu, a1[e], o);
      a2[e] += __shfl_xor_sync(0xffffffffu, a2[e], o);
    }
  }
  // element-major in shared memory (index (2e + which half) * LPR + lane): lanes of one
  // instruction hit different banks
  if ((threadIdx.x & 31) < LPR) {
#pragma unroll
    for (int e = 0; e < E; ++e) {
      atomicAdd(&s_dw[(2 * e) * LPR + lane], a1[e]);
      atomicAdd(&s_dw[(2 * e + 1) * LPR + lane], a2[e]);
    }
  }
  __syncthreads();
  float* my_ws = a.ws + static_cast<int64_t>(bid % dw_copies(N)) * N;
  for (int c = threadIdx.x; c < N; c += kThreads) {
    const int hsel = c >= half ? 1 : 0;
    const int cc = c - hsel * half;  // column inside its half: slice cc / E, element cc % E
    atomicAdd(my_ws + c, s_dw[(2 * (cc % E) + hsel) * LPR + cc / E]);
  }
  dw_finalize<T>(a.ws, static_cast<T*>(a.dw), N, nblk, threadIdx.x, kThreads);
}

bool mult_of(const int64_t* s, int n, int e) {
  for (int i = 0; i < n; ++i)
    if (s[i] % e != 0) return false;
  return true;
}

template <typename T, bool BWD>
bool side_ok(const HeadArgs& a) {
  constexpr int E = Cvt<T>::N;
  bool ok = aligned16(a.x) && aligned16(a.w) && aligned16(a.cos) && aligned16(a.sin) &&
            aligned16(a.out) && mult_of(a.xs, 3, E) && mult_of(a.os, 3, E) && mult_of(a.cs, 2, E);
  if (BWD) ok = ok && aligned16(a.dout) && mult_of(a.gs, 3, E);
  return ok;
}

template <typename T, bool BWD>
int launch_t(const HeadPair& pp, cudaStream_t s) {
  constexpr int E = Cvt<T>::N;
  const int D = pp.p[0].D;
  const int lpr = D / (2 * E);  // lanes per head row: each holds one slice of either half
  if (D % (2 * E) != 0 || !(lpr == 4 || lpr == 8 || lpr == 16) || !side_ok<T, BWD>(pp.p[0]) ||
      !side_ok<T, BWD>(pp.p[1])) {
    set_error("qk_norm_rope: head_dim %d with this element size / alignment is not supported "
              "(head rows of 128, 256 or 512 bytes, 16-byte aligned strides); run the norm and "
              "the rotation as separate calls",
              D);
    return BT_ERR_ARG;
  }
  constexpr int kHpi = BWD ? 2 : 4;  // heads per work item: 16-byte loads in flight per lane = 2 (4) * kHpi
  int64_t blocks[2];
  for (int i = 0; i < 2; ++i) {
    const HeadArgs& a = pp.p[i];
    const int64_t items = a.B * a.T * ceil_div(a.H, kHpi);
    if (items >= (1ll << 31) || a.B * a.T * a.H >= (1ll << 31)) {
      set_error("qk_norm_rope: %lld head rows exceed the 32-bit work index",
                (long long)(a.B * a.T * a.H));
      return BT_ERR_ARG;
    }
    blocks[i] = ceil_div(items, kThreads / lpr);
  }
  // The CTA budget is shared out in proportion to the work of the two sides.
  const int64_t cap = static_cast<int64_t>(sm_count()) * (BWD ? 2 : 8);
  int64_t g0 = blocks[0], g1 = blocks[1];
  if (g0 + g1 > cap) {
    g0 = cap * blocks[0] / (blocks[0] + blocks[1]);
    if (g0 < 1) g0 = 1;
    if (g0 > cap - 1) g0 = cap - 1;
    g1 = cap - g0;
    if (g0 > blocks[0]) g0 = blocks[0];
    if (g1 > blocks[1]) g1 = blocks[1];
  }
  HeadPair q = pp;
  q.split = static_cast<unsigned>(g0);
  const unsigned grid = static_cast<unsigned>(g0 + g1);
  cudaError_t le = cudaSuccess;
#define BT_HEAD(L)                                                         \
  if (lpr == L) {                                                          \
    if constexpr (BWD)                                                     \
      le = launch_dependent(headnorm_rope_bwd<T, L, kHpi, 2>, dim3(grid), dim3(kThreads), 0, s, q); \
    else                                                                   \
      le = launch_dependent(headnorm_rope_fwd<T, L, kHpi, 3>, dim3(grid), dim3(kThreads), 0, s, q); \
  }
  BT_HEAD(4)
  BT_HEAD(8)
  BT_HEAD(16)
#undef BT_HEAD
  BT_CHECK_LAUNCHED(le, BWD ? "headnorm_rope_bwd" : "headnorm_rope_fwd");
  return BT_OK;
}

template <bool BWD>
int launch_any(int dtype, const HeadPair& pp, cudaStream_t s) {
  switch (dtype) {
    case BT_BF16: return launch_t<__nv_bfloat16, BWD>(pp, s);
    case BT_FP16: return launch_t<__half, BWD>(pp, s);
    case BT_FP32: return launch_t<float, BWD>(pp, s);
  }
  set_error("qk_norm_rope: unknown dtype %d", dtype);
  return BT_ERR_ARG;
}

int check_common(const char* what, int64_t B, int64_t T, int64_t Hq, int64_t Hk, int64_t D,
                 int64_t cos_bs) {
  BT_CHECK_ARG(B >= 0 && T >= 0 && Hq >= 0 && Hk >= 0, "%s: negative size", what);
  BT_CHECK_ARG(D > 0 && D % 2 == 0 && D <= 4096, "%s: head_dim %lld must be even and <= 4096", what,
               (long long)D);
  BT_CHECK_ARG(cos_bs == 1 || cos_bs == B, "%s: cos batch %lld is neither 1 nor B=%lld", what,
               (long long)cos_bs, (long long)B);
  return BT_OK;
}

void fill_side(HeadArgs* a, int64_t B, int64_t T, int64_t H, int64_t D, const void* cos,
               const void* sin, const int64_t cos_strides[2], int64_t cos_bs) {
  a->B = B;
  a->T = T;
  a->H = H;
  a->D = static_cast<int>(D);
  a->cos = cos;
  a->sin = sin;
  a->cs[0] = cos_strides[0];
  a->cs[1] = cos_strides[1];
  a->cos_bs = static_cast<int>(cos_bs);
}

}  // namespace
}  // namespace bt

extern "C" int bt_qk_norm_rope_fwd(const void* q, const void* k, const void* wq, const void* wk,
                                   const void* cos, const void* sin, void* q_out, void* k_out,
                                   float* rstd_q, float* rstd_k, int64_t B, int64_t T, int64_t Hq,
                                   int64_t Hk, int64_t D, const int64_t q_strides[3],
                                   const int64_t k_strides[3], const int64_t q_out_strides[3],
                                   const int64_t k_out_strides[3], const int64_t cos_strides[2],
                                   int64_t cos_bs, float eps_q, float eps_k, int dtype,
                                   void* stream) {
  using namespace bt;
  if (int rc = check_common("qk_norm_rope_fwd", B, T, Hq, Hk, D, cos_bs)) return rc;
  if (B == 0 || T == 0) return BT_OK;
  BT_CHECK_ARG(Hq > 0 && Hk > 0, "qk_norm_rope_fwd: both q and k need at least one head");
  BT_CHECK_ARG(q && k && wq && wk && cos && sin && q_out && k_out && rstd_q && rstd_k,
               "qk_norm_rope_fwd: null pointer");
  HeadPair pp{};
  fill_side(&pp.p[0], B, T, Hq, D, cos, sin, cos_strides, cos_bs);
  fill_side(&pp.p[1], B, T, Hk, D, cos, sin, cos_strides, cos_bs);
  pp.p[0].x = q;
  pp.p[0].w = wq;
  pp.p[0].out = q_out;
  pp.p[0].rstd_out = rstd_q;
  pp.p[0].eps = eps_q;
  pp.p[1].x = k;
  pp.p[1].w = wk;
  pp.p[1].out = k_out;
  pp.p[1].rstd_out = rstd_k;
  pp.p[1].eps = eps_k;
  for (int i = 0; i < 3; ++i) {
    pp.p[0].xs[i] = q_strides[i];
    pp.p[0].os[i] = q_out_strides[i];
    pp.p[1].xs[i] = k_strides[i];
    pp.p[1].os[i] = k_out_strides[i];
  }
  return launch_any<false>(dtype, pp, static_cast<cudaStream_t>(stream));
}

extern "C" int bt_qk_norm_rope_bwd(const void* dq_out, const void* dk_out, const void* q,
                                   const void* k, const void* wq, const void* wk,
                                   const float* rstd_q, const float* rstd_k, const void* cos,
                                   const void* sin, void* dq, void* dk, void* dwq, void* dwk,
                                   void* ws_q, void* ws_k, int64_t B, int64_t T, int64_t Hq,
                                   int64_t Hk, int64_t D, const int64_t dq_out_strides[3],
                                   const int64_t dk_out_strides[3], const int64_t q_strides[3],
                                   const int64_t k_strides[3], const int64_t dq_strides[3],
                                   const int64_t dk_strides[3], const int64_t cos_strides[2],
                                   int64_t cos_bs, int dtype, void* stream) {
  using namespace bt;
  if (int rc = check_common("qk_norm_rope_bwd", B, T, Hq, Hk, D, cos_bs)) return rc;
  BT_CHECK_ARG(B > 0 && T > 0 && Hq > 0 && Hk > 0, "qk_norm_rope_bwd: empty input");
  BT_CHECK_ARG(dq_out && dk_out && q && k && wq && wk && rstd_q && rstd_k && cos && sin && dq &&
                   dk && dwq && dwk && ws_q && ws_k,
               "qk_norm_rope_bwd: null pointer");
  BT_CHECK_ARG(ws_q != ws_k, "qk_norm_rope_bwd: q and k need separate scratch buffers");
  HeadPair pp{};
  fill_side(&pp.p[0], B, T, Hq, D, cos, sin, cos_strides, cos_bs);
  fill_side(&pp.p[1], B, T, Hk, D, cos, sin, cos_strides, cos_bs);
  pp.p[0].dout = dq_out;
  pp.p[0].x = q;
  pp.p[0].w = wq;
  pp.p[0].rstd_in = rstd_q;
  pp.p[0].out = dq;
  pp.p[0].dw = dwq;
  pp.p[0].ws = static_cast<float*>(ws_q);
  pp.p[1].dout = dk_out;
  pp.p[1].x = k;
  pp.p[1].w = wk;
  pp.p[1].rstd_in = rstd_k;
  pp.p[1].out = dk;
  pp.p[1].dw = dwk;
  pp.p[1].ws = static_cast<float*>(ws_k);
  for (int i = 0; i < 3; ++i) {
    pp.p[0].gs[i] = dq_out_strides[i];
    pp.p[0].xs[i] = q_strides[i];
    pp.p[0].os[i] = dq_strides[i];
    pp.p[1].gs[i] = dk_out_strides[i];
    pp.p[1].xs[i] = k_strides[i];
    pp.p[1].os[i] = dk_strides[i];
  }
  return launch_any<true>(dtype, pp, static_cast<cudaStream_t>(stream));
}

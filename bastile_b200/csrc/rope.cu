// Rotate-half RoPE for sm_100a, forward (in place) and backward (sin negated,
// out of place on the incoming gradients).  Bandwidth-bound: every q/k element
// is read once and written once with 16-byte accesses; the cos/sin half rows
// (T x D/2) are shared by all heads and stay in L1/L2.
//
// Work decomposition: one thread owns one 16-byte column slice j of the first
// half and the matching slice of the second half, for one (batch, position) and
// a block of kHeadsPerThread heads, all of whose loads are issued before the
// first use.  q heads and k heads are one index space [0, Hq + Hk).
#include "bt_common.cuh"

namespace bt {
namespace {

constexpr int kThreads = 256;
constexpr int kHeadsPerThread = 4;

struct RopeArgs {
  const void* q_in;
  const void* k_in;
  void* q_out;
  void* k_out;
  const void* cos;
  const void* sin;
  int64_t B, Hq, Hk, T;
  int D;
  int64_t qi[3], ki[3], qo[3], ko[3];
  int64_t cs[2];
  int cos_bs;
  float sin_sign;
  int heads_fast;  // 1: consecutive lanes walk heads before positions
};

template <typename T>
__global__ void __launch_bounds__(kThreads) rope_vec(const RopeArgs a) {
  constexpr int E = Cvt<T>::N;
  grid_dependency_wait();
  const int half = a.D / 2;
  const int vph = half / E;  // vectors per half row
  const int64_t H = a.Hq + a.Hk;
  const int64_t hblocks = (H + kHeadsPerThread - 1) / kHeadsPerThread;
  const int64_t total = a.B * a.T * hblocks * vph;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * kThreads) {
    const int j = static_cast<int>(idx % vph);
    int64_t rest = idx / vph;
    int64_t t, hb;
    if (a.heads_fast) {
      hb = rest % hblocks;
      rest /= hblocks;
      t = rest % a.T;
      rest /= a.T;
    } else {
      t = rest % a.T;
      rest /= a.T;
      hb = rest % hblocks;
      rest /= hblocks;
    }
    const int64_t b = rest;
    const int64_t cb = (a.cos_bs == 1) ? 0 : b;
    const T* cp = static_cast<const T*>(a.cos) + cb * a.cs[0] + t * a.cs[1] + j * E;
    const T* sp = static_cast<const T*>(a.sin) + cb * a.cs[0] + t * a.cs[1] + j * E;
    const uint4 cv = ld_global_v4(cp);
    const uint4 sv = ld_global_v4(sp);

    uint4 v1[kHeadsPerThread], v2[kHeadsPerThread];
    T* outp[kHeadsPerThread];
#pragma unroll
    for (int u = 0; u < kHeadsPerThread; ++u) {
      const int64_t h = hb * kHeadsPerThread + u;
      outp[u] = nullptr;
      if (h < H) {
        const bool is_q = h < a.Hq;
        const int64_t hh = is_q ? h : h - a.Hq;
        const int64_t* si = is_q ? a.qi : a.ki;
        const int64_t* so = is_q ? a.qo : a.ko;
        const T* in = static_cast<const T*>(is_q ? a.q_in : a.k_in) + b * si[0] + hh * si[1] +
                      t * si[2] + j * E;
        outp[u] = static_cast<T*>(is_q ? a.q_out : a.k_out) + b * so[0] + hh * so[1] + t * so[2] +
                  j * E;
        v1[u] = ld_stream_v4(in);
        v2[u] = ld_stream_v4(in + half);
      }
    }
    float c[E], s[E];
    Cvt<T>::unpack(cv, c);
    Cvt<T>::unpack(sv, s);
#pragma unroll
    for (int e = 0; e < E; ++e) s[e] *= a.sin_sign;
#pragma unroll
    for (int u = 0; u < kHeadsPerThread; ++u) {
      if (outp[u] != nullptr) {
        float x1[E], x2[E], o1[E], o2[E];
        Cvt<T>::unpack(v1[u], x1);
        Cvt<T>::unpack(v2[u], x2);
#pragma unroll
        for (int e = 0; e < E; ++e) {
          // written out as explicit fused multiply-adds: the fused q/k-norm + RoPE kernels
          // use the same two operations and stay bit-identical to this one
          o1[e] = fmaf(-x2[e], s[e], x1[e] * c[e]);
          o2[e] = fmaf(x1[e], s[e], x2[e] * c[e]);
        }
        st_global_v4(outp[u], Cvt<T>::pack(o1));
        st_global_v4(outp[u] + half, Cvt<T>::pack(o2));
      }
    }
  }
}

// Any head_dim (even) / alignment: one element pair per thread.
template <typename T>
__global__ void __launch_bounds__(kThreads) rope_scalar(const RopeArgs a) {
  const int half = a.D / 2;
  const int64_t H = a.Hq + a.Hk;
  const int64_t total = a.B * H * a.T * half;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * kThreads) {
    const int j = static_cast<int>(idx % half);
    int64_t rest = idx / half;
    const int64_t t = rest % a.T;
    rest /= a.T;
    const int64_t h = rest % H;
    const int64_t b = rest / H;
    const int64_t cb = (a.cos_bs == 1) ? 0 : b;
    const float c = Cvt<T>::to_f(static_cast<const T*>(a.cos)[cb * a.cs[0] + t * a.cs[1] + j]);
    const float s =
        Cvt<T>::to_f(static_cast<const T*>(a.sin)[cb * a.cs[0] + t * a.cs[1] + j]) * a.sin_sign;
    const bool is_q = h < a.Hq;
    const int64_t hh = is_q ? h : h - a.Hq;
    const int64_t* si = is_q ? a.qi : a.ki;
    const int64_t* so = is_q ? a.qo : a.ko;
    const T* in =
        static_cast<const T*>(is_q ? a.q_in : a.k_in) + b * si[0] + hh * si[1] + t * si[2] + j;
    T* out = static_cast<T*>(is_q ? a.q_out : a.k_out) + b * so[0] + hh * so[1] + t * so[2] + j;
    const float x1 = Cvt<T>::to_f(in[0]);
    const float x2 = Cvt<T>::to_f(in[half]);
    out[0] = Cvt<T>::from_f(x1 * c - x2 * s);
    out[half] = Cvt<T>::from_f(x2 * c + x1 * s);
  }
}

bool strides_vec_ok(const int64_t s[3], int e) {
  return s[0] % e == 0 && s[1] % e == 0 && s[2] % e == 0;
}

template <typename T>
int launch(const RopeArgs& a, cudaStream_t s) {
  constexpr int E = Cvt<T>::N;
  const int half = a.D / 2;
  const int64_t H = a.Hq + a.Hk;
  const bool vec_ok = (half % E == 0) && aligned16(a.q_in) && aligned16(a.k_in) &&
                      aligned16(a.q_out) && aligned16(a.k_out) && aligned16(a.cos) &&
                      aligned16(a.sin) && strides_vec_ok(a.qi, E) && strides_vec_ok(a.ki, E) &&
                      strides_vec_ok(a.qo, E) && strides_vec_ok(a.ko, E) && a.cs[0] % E == 0 &&
                      a.cs[1] % E == 0;
  if (vec_ok) {
    const int64_t hblocks = (H + kHeadsPerThread - 1) / kHeadsPerThread;
    const int64_t total = a.B * a.T * hblocks * (half / E);
    const int64_t blocks = ceil_div(total, kThreads);
    // whole waves of the 3 CTAs an SM holds (16 per SM = 5.33 waves was 3 % slower)
    const int64_t cap = static_cast<int64_t>(sm_count()) * 12;
    BT_CHECK_LAUNCHED(launch_dependent(rope_vec<T>, dim3(static_cast<unsigned>(blocks < cap ? blocks : cap)),
                                       dim3(kThreads), 0, s, a),
                      "rope_vec");
  } else {
    const int64_t total = a.B * H * a.T * half;
    const int64_t blocks = ceil_div(total, kThreads);
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    rope_scalar<T><<<static_cast<unsigned>(blocks < cap ? blocks : cap), kThreads, 0, s>>>(a);
    BT_CHECK_LAUNCH("rope_scalar");
  }
  return BT_OK;
}

}  // namespace
}  // namespace bt

extern "C" int bt_rope(const void* q_in, const void* k_in, void* q_out, void* k_out,
                       const void* cos, const void* sin, int64_t B, int64_t Hq, int64_t Hk,
                       int64_t T, int64_t D, const int64_t q_in_strides[3],
                       const int64_t k_in_strides[3], const int64_t q_out_strides[3],
                       const int64_t k_out_strides[3], const int64_t cos_strides[2],
                       int64_t cos_bs, int negate_sin, int dtype, void* stream) {
  using namespace bt;
  BT_CHECK_ARG(B >= 0 && Hq >= 0 && Hk >= 0 && T >= 0, "rope: negative size");
  BT_CHECK_ARG(D > 0 && D % 2 == 0 && D < (1 << 20), "rope: head_dim %lld must be even",
               (long long)D);
  BT_CHECK_ARG(cos_bs == 1 || cos_bs == B, "rope: cos batch %lld is neither 1 nor B=%lld",
               (long long)cos_bs, (long long)B);
  if (B == 0 || T == 0 || Hq + Hk == 0) return BT_OK;
  BT_CHECK_ARG(cos && sin, "rope: null cos/sin");
  BT_CHECK_ARG(Hq == 0 || (q_in && q_out), "rope: null q");
  BT_CHECK_ARG(Hk == 0 || (k_in && k_out), "rope: null k");
  RopeArgs a{};
  a.q_in = q_in;
  a.k_in = k_in;
  a.q_out = q_out;
  a.k_out = k_out;
  a.cos = cos;
  a.sin = sin;
  a.B = B;
  a.Hq = Hq;
  a.Hk = Hk;
  a.T = T;
  a.D = static_cast<int>(D);
  for (int i = 0; i < 3; ++i) {
    a.qi[i] = q_in_strides[i];
    a.ki[i] = k_in_strides[i];
    a.qo[i] = q_out_strides[i];
    a.ko[i] = k_out_strides[i];
  }
  a.cs[0] = cos_strides[0];
  a.cs[1] = cos_strides[1];
  a.cos_bs = static_cast<int>(cos_bs);
  a.sin_sign = negate_sin ? -1.0f : 1.0f;
  // Walk heads first when heads are closer together in memory than positions
  // ([B,T,H,D] storage viewed as [B,H,T,D], the layout HF attention hands over).
  const int64_t* ref = Hq > 0 ? q_in_strides : k_in_strides;
  a.heads_fast = (ref[1] < ref[2]) ? 1 : 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case BT_BF16: return launch<__nv_bfloat16>(a, s);
    case BT_FP16: return launch<__half>(a, s);
    case BT_FP32: return launch<float>(a, s);
  }
  set_error("rope: unknown dtype %d", dtype);
  return BT_ERR_ARG;
}

// AdamW step for sm_100a: one streaming pass over (param, grad, exp_avg, exp_avg_sq) per
// tensor - 4 reads and 3 writes of 16-byte vectors per 8 (16-bit) or 4 (fp32) elements, fp32
// arithmetic, results rounded once to the storage type.  Large tensors get a launch of their
// own; small ones (norm weights) are batched so that a 36-layer model does not pay a launch
// per 4096-element vector.
//
// Update (decoupled weight decay, as torch.optim.AdamW):
//   p  <- p * (1 - lr * wd)
//   m  <- beta1 * m + (1 - beta1) * g
//   v  <- beta2 * v + (1 - beta2) * g * g
//   p  <- p - (lr / bc1) * m / (sqrt(v) / sqrt(bc2) + eps)      bc_i = 1 - beta_i^step
#include "bt_common.cuh"

namespace bt {
namespace {

constexpr int kThreads = 256;
constexpr int kBatch = 48;  // tensors per batched launch (pointer table lives in kernel params)

struct Hyper {
  float lr, beta1, beta2, eps, wd, inv_bc1, inv_sqrt_bc2;
};

// U 16-byte vectors per thread, `stride` vectors apart: all 4*U loads are issued before the
// first use.
template <typename T, int U>
__device__ __forceinline__ void update_vecs(T* __restrict__ p, const T* __restrict__ g,
                                            T* __restrict__ m, T* __restrict__ v, int64_t first,
                                            int64_t stride, const Hyper& h) {
  constexpr int E = Cvt<T>::N;
  uint4 pr[U], gr[U], mr[U], vr[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int64_t off = (first + u * stride) * E;
    pr[u] = ld_stream_v4(p + off);
    gr[u] = ld_stream_v4(g + off);
    mr[u] = ld_stream_v4(m + off);
    vr[u] = ld_stream_v4(v + off);
  }
  const float decay = 1.0f - h.lr * h.wd;
  const float step = h.lr * h.inv_bc1;
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int64_t off = (first + u * stride) * E;
    float pf[E], gf[E], mf[E], vf[E];
    Cvt<T>::unpack(pr[u], pf);
    Cvt<T>::unpack(gr[u], gf);
    Cvt<T>::unpack(mr[u], mf);
    Cvt<T>::unpack(vr[u], vf);
#pragma unroll
    for (int e = 0; e < E; ++e) {
      mf[e] = h.beta1 * mf[e] + (1.0f - h.beta1) * gf[e];
      vf[e] = h.beta2 * vf[e] + (1.0f - h.beta2) * gf[e] * gf[e];
      const float denom = sqrtf(vf[e]) * h.inv_sqrt_bc2 + h.eps;
      pf[e] = pf[e] * decay - step * (mf[e] / denom);
    }
    st_global_v4(p + off, Cvt<T>::pack(pf));
    st_global_v4(m + off, Cvt<T>::pack(mf));
    st_global_v4(v + off, Cvt<T>::pack(vf));
  }
}

template <typename T>
__device__ __forceinline__ void update_scalar(T* p, const T* g, T* m, T* v, int64_t i,
                                              const Hyper& h) {
  const float gf = Cvt<T>::to_f(g[i]);
  const float mf = h.beta1 * Cvt<T>::to_f(m[i]) + (1.0f - h.beta1) * gf;
  const float vf = h.beta2 * Cvt<T>::to_f(v[i]) + (1.0f - h.beta2) * gf * gf;
  const float denom = sqrtf(vf) * h.inv_sqrt_bc2 + h.eps;
  const float pf = Cvt<T>::to_f(p[i]) * (1.0f - h.lr * h.wd) - h.lr * h.inv_bc1 * (mf / denom);
  p[i] = Cvt<T>::from_f(pf);
  m[i] = Cvt<T>::from_f(mf);
  v[i] = Cvt<T>::from_f(vf);
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
adamw_one(T* __restrict__ p, const T* __restrict__ g, T* __restrict__ m, T* __restrict__ v,
          int64_t n, int vec_ok, Hyper h) {
  constexpr int E = Cvt<T>::N;
  grid_dependency_wait();
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  const int64_t nvec = vec_ok ? n / E : 0;
  // one vector per thread per pass measured faster than two in flight (occupancy covers the latency)
  for (int64_t i = tid; i < nvec; i += stride) update_vecs<T, 1>(p, g, m, v, i, stride, h);
  for (int64_t i = nvec * E + tid; i < n; i += stride) update_scalar<T>(p, g, m, v, i, h);
}

struct Table {
  void* p[kBatch];
  const void* g[kBatch];
  void* m[kBatch];
  void* v[kBatch];
  int64_t n[kBatch];
  int count;
};

// blockIdx.y = tensor; blockIdx.x strides over it (scalar accesses: these tensors are small)
template <typename T>
__global__ void __launch_bounds__(kThreads) adamw_many(const Table t, Hyper h) {
  const int k = blockIdx.y;
  if (k >= t.count) return;
  T* p = static_cast<T*>(t.p[k]);
  const T* g = static_cast<const T*>(t.g[k]);
  T* m = static_cast<T*>(t.m[k]);
  T* v = static_cast<T*>(t.v[k]);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < t.n[k];
       i += static_cast<int64_t>(gridDim.x) * kThreads)
    update_scalar<T>(p, g, m, v, i, h);
}

template <typename T>
int one_t(void* p, const void* g, void* m, void* v, int64_t n, const Hyper& h, int ctas_per_sm,
          cudaStream_t s) {
  constexpr int E = Cvt<T>::N;
  const int vec_ok = aligned16(p) && aligned16(g) && aligned16(m) && aligned16(v);
  const int64_t work = vec_ok ? ceil_div(n, E) : n;
  const int64_t blocks = ceil_div(work, kThreads);
  const int64_t cap = static_cast<int64_t>(sm_count()) * ctas_per_sm;
  BT_CHECK_LAUNCHED(
      launch_dependent(adamw_one<T>, dim3(static_cast<unsigned>(blocks < 1 ? 1 : (blocks < cap ? blocks : cap))),
                       dim3(kThreads), 0, s, static_cast<T*>(p), static_cast<const T*>(g), static_cast<T*>(m),
                       static_cast<T*>(v), n, vec_ok, h),
      "adamw_one");
  return BT_OK;
}

template <typename T>
int many_t(const Table& t, int64_t max_n, const Hyper& h, cudaStream_t s) {
  int64_t bx = ceil_div(max_n, kThreads);
  if (bx > 64) bx = 64;
  if (bx < 1) bx = 1;
  adamw_many<T><<<dim3(static_cast<unsigned>(bx), static_cast<unsigned>(t.count)), kThreads, 0, s>>>(t, h);
  BT_CHECK_LAUNCH("adamw_many");
  return BT_OK;
}

// ---- fp32 master weights --------------------------------------------------------------
// The optimizer state (master parameter, both moments) is fp32; the gradient arrives in the
// model's 16-bit (or fp32) type T and the updated parameter is also written back in T for the
// next forward pass.  Per element: 3 fp32 reads + 1 T read, 3 fp32 writes + 1 T write.
template <typename T>
__global__ void __launch_bounds__(kThreads)
adamw_master(float* __restrict__ p32, float* __restrict__ m, float* __restrict__ v,
             const T* __restrict__ g, T* __restrict__ p_out, int64_t n, int vec_ok, float gscale,
             Hyper h) {
  constexpr int E = Cvt<T>::N;   // elements per 16-byte vector of T
  constexpr int Q = E / 4;       // float4 vectors of fp32 state per vector of T
  grid_dependency_wait();
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  const int64_t nvec = vec_ok ? n / E : 0;
  const float decay = 1.0f - h.lr * h.wd;
  const float step = h.lr * h.inv_bc1;
  for (int64_t i = tid; i < nvec; i += stride) {
    const int64_t off = i * E;
    uint4 pr[Q], mr[Q], vr[Q];
    const uint4 gr = ld_stream_v4(g + off);
#pragma unroll
    for (int q = 0; q < Q; ++q) {
      pr[q] = ld_stream_v4(p32 + off + 4 * q);
      mr[q] = ld_stream_v4(m + off + 4 * q);
      vr[q] = ld_stream_v4(v + off + 4 * q);
    }
    float gf[E], out[E];
    Cvt<T>::unpack(gr, gf);
#pragma unroll
    for (int q = 0; q < Q; ++q) {
      float pf[4], mf[4], vf[4];
      Cvt<float>::unpack(pr[q], pf);
      Cvt<float>::unpack(mr[q], mf);
      Cvt<float>::unpack(vr[q], vf);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float ge = gf[4 * q + e] * gscale;
        mf[e] = h.beta1 * mf[e] + (1.0f - h.beta1) * ge;
        vf[e] = h.beta2 * vf[e] + (1.0f - h.beta2) * ge * ge;
        const float denom = sqrtf(vf[e]) * h.inv_sqrt_bc2 + h.eps;
        pf[e] = pf[e] * decay - step * (mf[e] / denom);
        out[4 * q + e] = pf[e];
      }
      st_global_v4(p32 + off + 4 * q, Cvt<float>::pack(pf));
      st_global_v4(m + off + 4 * q, Cvt<float>::pack(mf));
      st_global_v4(v + off + 4 * q, Cvt<float>::pack(vf));
    }
    st_global_v4(p_out + off, Cvt<T>::pack(out));
  }
  for (int64_t i = nvec * E + tid; i < n; i += stride) {
    const float ge = Cvt<T>::to_f(g[i]) * gscale;
    const float mf = h.beta1 * m[i] + (1.0f - h.beta1) * ge;
    const float vf = h.beta2 * v[i] + (1.0f - h.beta2) * ge * ge;
    const float denom = sqrtf(vf) * h.inv_sqrt_bc2 + h.eps;
    const float pf = p32[i] * decay - step * (mf / denom);
    p32[i] = pf;
    m[i] = mf;
    v[i] = vf;
    p_out[i] = Cvt<T>::from_f(pf);
  }
}

template <typename T>
int master_t(float* p32, float* m, float* v, const void* g, void* p_out, int64_t n, float gscale,
             const Hyper& h, int ctas_per_sm, cudaStream_t s) {
  constexpr int E = Cvt<T>::N;
  const int vec_ok = aligned16(p32) && aligned16(m) && aligned16(v) && aligned16(g) && aligned16(p_out);
  const int64_t work = vec_ok ? ceil_div(n, E) : n;
  const int64_t blocks = ceil_div(work, kThreads);
  const int64_t cap = static_cast<int64_t>(sm_count()) * ctas_per_sm;
  BT_CHECK_LAUNCHED(
      launch_dependent(adamw_master<T>, dim3(static_cast<unsigned>(blocks < 1 ? 1 : (blocks < cap ? blocks : cap))),
                       dim3(kThreads), 0, s, p32, m, v, static_cast<const T*>(g), static_cast<T*>(p_out), n,
                       vec_ok, gscale, h),
      "adamw_master");
  return BT_OK;
}

Hyper make_hyper(float lr, float beta1, float beta2, float eps, float weight_decay, int64_t step) {
  Hyper h;
  h.lr = lr;
  h.beta1 = beta1;
  h.beta2 = beta2;
  h.eps = eps;
  h.wd = weight_decay;
  h.inv_bc1 = static_cast<float>(1.0 / (1.0 - pow(static_cast<double>(beta1), static_cast<double>(step))));
  h.inv_sqrt_bc2 =
      static_cast<float>(1.0 / sqrt(1.0 - pow(static_cast<double>(beta2), static_cast<double>(step))));
  return h;
}

}  // namespace
}  // namespace bt

extern "C" int bt_adamw_step(void* const* params, const void* const* grads, void* const* exp_avg,
                             void* const* exp_avg_sq, const int64_t* numel, int n_tensors, float lr,
                             float beta1, float beta2, float eps, float weight_decay, int64_t step,
                             int ctas_per_sm, int dtype, void* stream) {
  using namespace bt;
  BT_CHECK_ARG(n_tensors >= 0 && step >= 1, "adamw_step: bad tensor count or step");
  BT_CHECK_ARG(ctas_per_sm >= 0 && ctas_per_sm <= 32, "adamw_step: ctas_per_sm must be 0..32");
  if (ctas_per_sm == 0) ctas_per_sm = 16;
  BT_CHECK_ARG(n_tensors == 0 || (params && grads && exp_avg && exp_avg_sq && numel),
               "adamw_step: null table");
  BT_CHECK_ARG(dtype == BT_BF16 || dtype == BT_FP16 || dtype == BT_FP32, "adamw_step: unknown dtype %d",
               dtype);
  const Hyper h = make_hyper(lr, beta1, beta2, eps, weight_decay, step);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  constexpr int64_t kSmall = 1 << 16;  // tensors up to 64 Ki elements are batched
  Table t;
  t.count = 0;
  int64_t max_n = 0;
  auto flush = [&]() -> int {
    if (t.count == 0) return BT_OK;
    int rc = BT_OK;
    switch (dtype) {
      case BT_BF16: rc = many_t<__nv_bfloat16>(t, max_n, h, s); break;
      case BT_FP16: rc = many_t<__half>(t, max_n, h, s); break;
      default: rc = many_t<float>(t, max_n, h, s); break;
    }
    t.count = 0;
    max_n = 0;
    return rc;
  };
  for (int i = 0; i < n_tensors; ++i) {
    const int64_t n = numel[i];
    if (n <= 0) continue;
    BT_CHECK_ARG(params[i] && grads[i] && exp_avg[i] && exp_avg_sq[i], "adamw_step: null tensor %d", i);
    if (n <= kSmall) {
      t.p[t.count] = params[i];
      t.g[t.count] = grads[i];
      t.m[t.count] = exp_avg[i];
      t.v[t.count] = exp_avg_sq[i];
      t.n[t.count] = n;
      max_n = n > max_n ? n : max_n;
      if (++t.count == kBatch) {
        if (int rc = flush()) return rc;
      }
      continue;
    }
    int rc;
    switch (dtype) {
      case BT_BF16: rc = one_t<__nv_bfloat16>(params[i], grads[i], exp_avg[i], exp_avg_sq[i], n, h, ctas_per_sm, s); break;
      case BT_FP16: rc = one_t<__half>(params[i], grads[i], exp_avg[i], exp_avg_sq[i], n, h, ctas_per_sm, s); break;
      default: rc = one_t<float>(params[i], grads[i], exp_avg[i], exp_avg_sq[i], n, h, ctas_per_sm, s); break;
    }
    if (rc) return rc;
  }
  return flush();
}

extern "C" int bt_adamw_master_step(float* master, float* exp_avg, float* exp_avg_sq, const void* grad,
                                    void* param_out, int64_t numel, float lr, float beta1, float beta2,
                                    float eps, float weight_decay, int64_t step, float grad_scale,
                                    int ctas_per_sm, int dtype, void* stream) {
  using namespace bt;
  BT_CHECK_ARG(numel >= 0 && step >= 1, "adamw_master_step: bad element count or step");
  BT_CHECK_ARG(ctas_per_sm >= 0 && ctas_per_sm <= 32, "adamw_master_step: ctas_per_sm must be 0..32");
  if (ctas_per_sm == 0) ctas_per_sm = 16;
  BT_CHECK_ARG(dtype == BT_BF16 || dtype == BT_FP16 || dtype == BT_FP32,
               "adamw_master_step: unknown dtype %d", dtype);
  if (numel == 0) return BT_OK;
  BT_CHECK_ARG(master && exp_avg && exp_avg_sq && grad && param_out, "adamw_master_step: null pointer");
  const Hyper h = make_hyper(lr, beta1, beta2, eps, weight_decay, step);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case BT_BF16:
      return master_t<__nv_bfloat16>(master, exp_avg, exp_avg_sq, grad, param_out, numel, grad_scale, h, ctas_per_sm, s);
    case BT_FP16:
      return master_t<__half>(master, exp_avg, exp_avg_sq, grad, param_out, numel, grad_scale, h, ctas_per_sm, s);
    default:
      return master_t<float>(master, exp_avg, exp_avg_sq, grad, param_out, numel, grad_scale, h, ctas_per_sm, s);
  }
}

// Streaming kernels around the logits GEMM of the fused cross-entropy: merging the
// per-tile softmax statistics, turning the logits chunk into scaled gradients in
// place, counting valid labels, reducing the loss, and the dloss scaling.
// None of them synchronises with the host.
#include "bt_common.cuh"

namespace bt {
namespace {

constexpr int kThreads = 256;

// One warp per row: (max, sum) over the row's column tiles, plus the target logit.
__global__ void __launch_bounds__(kThreads)
lce_row_stats_kernel(const float2* __restrict__ tile_stats, const float* __restrict__ tgt_logit,
                     float* __restrict__ row_stats, int64_t rows, int n_vt) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * kThreads) >> 5;
  for (int64_t row = warp0; row < rows; row += nwarps) {
    const float2* ts = tile_stats + row * n_vt;
    float mx = -1e30f, sum = 0.f;
    for (int i = lane; i < n_vt; i += 32) {
      const float2 t = ts[i];
      const float nm = fmaxf(mx, t.x);
      sum = sum * __expf(mx - nm) + t.y * __expf(t.x - nm);
      mx = nm;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float omx = __shfl_xor_sync(0xffffffffu, mx, o);
      const float osum = __shfl_xor_sync(0xffffffffu, sum, o);
      const float nm = fmaxf(mx, omx);
      sum = sum * __expf(mx - nm) + osum * __expf(omx - nm);
      mx = nm;
    }
    if (lane == 0) {
      row_stats[row * 3 + 0] = mx;
      row_stats[row * 3 + 1] = sum;
      row_stats[row * 3 + 2] = tgt_logit[row];
    }
  }
}

// Merge of the per-shard statistics of a vocabulary-parallel loss: shard_stats is
// [n_shards][rows][3] = (max, sum exp, target logit or 0) as gathered from the ranks; the
// result [rows][3] describes the full vocabulary (one thread per row).
__global__ void __launch_bounds__(kThreads)
lce_stats_combine_kernel(const float* __restrict__ shard_stats, float* __restrict__ row_stats,
                         int64_t rows, int64_t shard_stride, int n_shards) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (row >= rows) return;
  float mx = -1e30f;
  for (int s = 0; s < n_shards; ++s) mx = fmaxf(mx, shard_stats[s * shard_stride + row * 3]);
  float sum = 0.f, tgt = 0.f;
  for (int s = 0; s < n_shards; ++s) {
    const float* st = shard_stats + s * shard_stride + row * 3;
    sum += st[1] * __expf(st[0] - mx);
    tgt += st[2];
  }
  row_stats[row * 3 + 0] = mx;
  row_stats[row * 3 + 1] = sum;
  row_stats[row * 3 + 2] = tgt;
}

// logits[row, :] -> (softmax - onehot) * scale in place; one CTA walks whole rows so the
// row's statistics and label are read once.  Also writes the per-row loss.
template <typename T>
__global__ void __launch_bounds__(kThreads)
lce_dlogits_kernel(T* __restrict__ logits, const float* __restrict__ row_stats,
                   const int64_t* __restrict__ labels, float* __restrict__ loss_row,
                   const float* __restrict__ grad_scale, int64_t rows, int64_t V, int64_t ld,
                   int64_t v_offset, int64_t ignore_index, int write_loss) {
  constexpr int E = Cvt<T>::N;
  const float scale = __ldg(grad_scale);
  const int64_t nvec = (V + E - 1) / E;
  // gridDim.y splits a row into column segments so that few long rows still fill the GPU
  const int64_t seg = (nvec + gridDim.y - 1) / gridDim.y;
  const int64_t v_begin = static_cast<int64_t>(blockIdx.y) * seg;
  const int64_t v_end = v_begin + seg < nvec ? v_begin + seg : nvec;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float mx = row_stats[row * 3 + 0];
    const float sum = row_stats[row * 3 + 1];
    const int64_t label = labels[row];
    const bool valid = label != ignore_index;
    if (write_loss && blockIdx.y == 0 && threadIdx.x == 0)
      loss_row[row] = valid ? (mx + __logf(sum) - row_stats[row * 3 + 2]) : 0.f;
    const int64_t tcol = valid ? label - v_offset : -1;
    const float inv = scale / sum;
    T* lr = logits + row * ld;
    for (int64_t v = v_begin + threadIdx.x; v < v_end; v += kThreads) {
      const int64_t c0 = v * E;
      float f[E];
      if (valid) {
        Cvt<T>::unpack(ld_stream_v4(lr + c0), f);
#pragma unroll
        for (int e = 0; e < E; ++e) f[e] = __expf(f[e] - mx) * inv;
        if (tcol >= c0 && tcol < c0 + E) {
#pragma unroll
          for (int e = 0; e < E; ++e)
            if (c0 + e == tcol) f[e] -= scale;
        }
      } else {
#pragma unroll
        for (int e = 0; e < E; ++e) f[e] = 0.f;
      }
      // Columns >= V inside the last vector are row padding (ld is a multiple of E).
      st_global_v4(lr + c0, Cvt<T>::pack(f));
    }
  }
}

__global__ void __launch_bounds__(kThreads)
lce_count_valid_kernel(const int64_t* __restrict__ labels, int64_t n, int64_t ignore_index,
                       int mean, float* __restrict__ n_valid, float* __restrict__ grad_scale,
                       int64_t vocab, int32_t* __restrict__ status) {
  __shared__ unsigned long long s_cnt[kThreads / 32];
  unsigned long long c = 0;
  bool bad = false;
  for (int64_t i = threadIdx.x; i < n; i += kThreads) {
    const int64_t l = labels[i];
    c += (l != ignore_index) ? 1ull : 0ull;
    bad |= (l != ignore_index) && (l < 0 || l >= vocab);
  }
  // a label that is neither ignore_index nor a vocabulary row (F.cross_entropy asserts on it)
  if (vocab > 0 && status != nullptr && __syncthreads_or(bad) && threadIdx.x == 0)
    atomicOr(status, BT_STATUS_BAD_LABEL);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0) s_cnt[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long t = 0;
    for (int i = 0; i < kThreads / 32; ++i) t += s_cnt[i];
    const float nv = static_cast<float>(t);
    n_valid[0] = nv;
    grad_scale[0] = mean ? (t > 0 ? 1.0f / nv : 0.0f) : 1.0f;
  }
}

__global__ void __launch_bounds__(kThreads)
lce_reduce_loss_kernel(const float* __restrict__ loss_row, int64_t n,
                       const float* __restrict__ grad_scale, float* __restrict__ loss) {
  __shared__ double s_sum[kThreads / 32];
  double a = 0.0;
  for (int64_t i = threadIdx.x; i < n; i += kThreads) a += static_cast<double>(loss_row[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
  if ((threadIdx.x & 31) == 0) s_sum[threadIdx.x >> 5] = a;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int i = 0; i < kThreads / 32; ++i) t += s_sum[i];
    const float sc = grad_scale != nullptr ? grad_scale[0] : 1.0f;
    loss[0] = static_cast<float>(t * static_cast<double>(sc));
  }
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(kThreads)
scale_cast_kernel(const TI* __restrict__ in, TO* __restrict__ out, int64_t n,
                  const float* __restrict__ scale) {
  const float s = __ldg(scale);
  // 8 elements per thread per step: one 16-byte vector of a 16-bit type, two of fp32
  const int64_t nvec = n / 8;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; v < nvec; v += stride) {
    float f[8];
    if constexpr (sizeof(TI) == 4) {
      const float4 a = *reinterpret_cast<const float4*>(in + v * 8);
      const float4 b = *reinterpret_cast<const float4*>(in + v * 8 + 4);
      f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
      f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    } else {
      Cvt<TI>::unpack(ld_global_v4(in + v * 8), f);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] *= s;
    if constexpr (sizeof(TO) == 4) {
      *reinterpret_cast<float4*>(out + v * 8) = make_float4(f[0], f[1], f[2], f[3]);
      *reinterpret_cast<float4*>(out + v * 8 + 4) = make_float4(f[4], f[5], f[6], f[7]);
    } else {
      st_global_v4(out + v * 8, Cvt<TO>::pack(f));
    }
  }
  // tail
  for (int64_t i = nvec * 8 + static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n;
       i += stride)
    out[i] = Cvt<TO>::from_f(Cvt<TI>::to_f(in[i]) * s);
}

template <typename TI, typename TO>
int scale_cast_t(const void* in, void* out, int64_t n, const float* scale, cudaStream_t s) {
  const int64_t blocks = ceil_div(ceil_div(n, 8), kThreads);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  scale_cast_kernel<TI, TO><<<static_cast<unsigned>(blocks < 1 ? 1 : (blocks < cap ? blocks : cap)),
                              kThreads, 0, s>>>(static_cast<const TI*>(in), static_cast<TO*>(out),
                                                n, scale);
  BT_CHECK_LAUNCH("scale_cast");
  return BT_OK;
}

template <typename TI>
int scale_cast_in(const void* in, void* out, int64_t n, const float* scale, int out_dtype,
                  cudaStream_t s) {
  switch (out_dtype) {
    case BT_BF16: return scale_cast_t<TI, __nv_bfloat16>(in, out, n, scale, s);
    case BT_FP16: return scale_cast_t<TI, __half>(in, out, n, scale, s);
    case BT_FP32: return scale_cast_t<TI, float>(in, out, n, scale, s);
  }
  set_error("scale_cast: unknown output dtype %d", out_dtype);
  return BT_ERR_ARG;
}

}  // namespace
}  // namespace bt

extern "C" int bt_lce_row_stats(const float* tile_stats, const float* tgt_logit, float* row_stats,
                                int64_t rows, int64_t n_vtiles, void* stream) {
  using namespace bt;
  BT_CHECK_ARG(rows >= 0 && n_vtiles > 0 && n_vtiles < (1ll << 31), "lce_row_stats: bad sizes");
  if (rows == 0) return BT_OK;
  BT_CHECK_ARG(tile_stats && tgt_logit && row_stats, "lce_row_stats: null pointer");
  const int64_t blocks = ceil_div(rows, kThreads / 32);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  lce_row_stats_kernel<<<static_cast<unsigned>(blocks < cap ? blocks : cap), kThreads, 0,
                         static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float2*>(tile_stats), tgt_logit, row_stats, rows,
      static_cast<int>(n_vtiles));
  BT_CHECK_LAUNCH("lce_row_stats");
  return BT_OK;
}

extern "C" int bt_lce_dlogits(void* logits, const float* row_stats, const int64_t* labels,
                              float* loss_row, const float* grad_scale, int64_t rows, int64_t V,
                              int64_t ld_logits, int64_t v_offset, int64_t ignore_index,
                              int write_loss, int dtype, void* stream) {
  using namespace bt;
  BT_CHECK_ARG(rows >= 0 && V > 0, "lce_dlogits: bad sizes");
  if (rows == 0) return BT_OK;
  BT_CHECK_ARG(logits && row_stats && labels && grad_scale && (!write_loss || loss_row),
               "lce_dlogits: null pointer");
  BT_CHECK_ARG(dtype == BT_BF16 || dtype == BT_FP16 || dtype == BT_FP32, "lce_dlogits: unknown dtype");
  const int64_t vec = dtype == BT_FP32 ? 4 : 8;
  BT_CHECK_ARG(aligned16(logits) && ld_logits % vec == 0 && ld_logits >= (V + vec - 1) / vec * vec,
               "lce_dlogits: logits rows must be 16-byte aligned and padded to whole 16-byte vectors");
  const int sms = sm_count();
  // enough CTAs for ~8 per SM: split rows into column segments when there are few rows
  int64_t gx = rows < static_cast<int64_t>(sms) * 8 ? rows : static_cast<int64_t>(sms) * 8;
  int64_t gy = 1;
  const int64_t nvec = (V + 7) / 8;
  while (gx * gy < static_cast<int64_t>(sms) * 4 && gy * 2 * kThreads <= nvec) gy *= 2;
  dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == BT_BF16)
    lce_dlogits_kernel<__nv_bfloat16><<<grid, kThreads, 0, s>>>(
        static_cast<__nv_bfloat16*>(logits), row_stats, labels, loss_row, grad_scale, rows, V,
        ld_logits, v_offset, ignore_index, write_loss);
  else if (dtype == BT_FP16)
    lce_dlogits_kernel<__half><<<grid, kThreads, 0, s>>>(static_cast<__half*>(logits), row_stats,
                                                         labels, loss_row, grad_scale, rows, V,
                                                         ld_logits, v_offset, ignore_index,
                                                         write_loss);
  else
    lce_dlogits_kernel<float><<<grid, kThreads, 0, s>>>(static_cast<float*>(logits), row_stats,
                                                        labels, loss_row, grad_scale, rows, V,
                                                        ld_logits, v_offset, ignore_index,
                                                        write_loss);
  BT_CHECK_LAUNCH("lce_dlogits");
  return BT_OK;
}

extern "C" int bt_lce_stats_combine(const float* shard_stats, float* row_stats, int64_t rows,
                                    int64_t shard_stride, int n_shards, void* stream) {
  using namespace bt;
  BT_CHECK_ARG(rows >= 0 && n_shards >= 1 && shard_stride >= rows * 3, "lce_stats_combine: bad extents");
  if (rows == 0) return BT_OK;
  BT_CHECK_ARG(shard_stats && row_stats, "lce_stats_combine: null pointer");
  lce_stats_combine_kernel<<<static_cast<unsigned>(ceil_div(rows, kThreads)), kThreads, 0,
                             static_cast<cudaStream_t>(stream)>>>(shard_stats, row_stats, rows,
                                                                  shard_stride, n_shards);
  BT_CHECK_LAUNCH("lce_stats_combine");
  return BT_OK;
}

extern "C" int bt_lce_count_valid(const int64_t* labels, int64_t n, int64_t ignore_index, int mean,
                                  float* n_valid, float* grad_scale, int64_t vocab_size, int32_t* status,
                                  void* stream) {
  using namespace bt;
  BT_CHECK_ARG(n >= 0 && n_valid && grad_scale && (n == 0 || labels), "lce_count_valid: bad args");
  lce_count_valid_kernel<<<1, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      labels, n, ignore_index, mean, n_valid, grad_scale, vocab_size, status);
  BT_CHECK_LAUNCH("lce_count_valid");
  return BT_OK;
}

extern "C" int bt_lce_reduce_loss(const float* loss_row, int64_t n, const float* grad_scale,
                                  float* loss, void* stream) {
  using namespace bt;
  BT_CHECK_ARG(n >= 0 && loss && (n == 0 || loss_row), "lce_reduce_loss: bad args");
  lce_reduce_loss_kernel<<<1, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(loss_row, n,
                                                                               grad_scale, loss);
  BT_CHECK_LAUNCH("lce_reduce_loss");
  return BT_OK;
}

extern "C" int bt_scale_cast(const void* in, void* out, int64_t n, const float* scale, int in_dtype,
                             int out_dtype, void* stream) {
  using namespace bt;
  BT_CHECK_ARG(n >= 0, "scale_cast: negative size");
  if (n == 0) return BT_OK;
  BT_CHECK_ARG(in && out && scale, "scale_cast: null pointer");
  BT_CHECK_ARG(aligned16(in) && aligned16(out), "scale_cast: buffers must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (in_dtype) {
    case BT_BF16: return scale_cast_in<__nv_bfloat16>(in, out, n, scale, out_dtype, s);
    case BT_FP16: return scale_cast_in<__half>(in, out, n, scale, out_dtype, s);
    case BT_FP32: return scale_cast_in<float>(in, out, n, scale, out_dtype, s);
  }
  set_error("scale_cast: unknown input dtype %d", in_dtype);
  return BT_ERR_ARG;
}

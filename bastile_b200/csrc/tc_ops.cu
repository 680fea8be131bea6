// C entry points that run on the tcgen05 GEMM core: the plain GEMM, the fused
// SwiGLU MLP forward / backward and the logits + softmax-statistics step of the
// fused cross-entropy.
#include "gemm_sm100.cuh"

namespace bt {
namespace {

using gemm::Launch;
using gemm::Operand;

// operand storage the tensor-core kernels take: 16-bit floats, or fp32 read as tf32
bool is_tc(int dtype) { return dtype == BT_BF16 || dtype == BT_FP16 || dtype == BT_FP32; }
int esize(int dtype) { return dtype == BT_FP32 ? 4 : 2; }

Operand operand(const void* ptr, bool kmajor, int64_t mn, int64_t k, int64_t ld) {
  Operand o;
  o.ptr = ptr;
  o.kmajor = kmajor ? 1 : 0;
  o.mn = mn;
  o.k = k;
  o.ld = ld;
  return o;
}

bool rows_aligned(const void* p, int64_t ld, int elem_bytes) {
  return p == nullptr || (aligned16(p) && (ld * elem_bytes) % 16 == 0);
}

int check_dims(const char* what, int64_t m, int64_t n, int64_t k) {
  if (m <= 0 || n <= 0 || k <= 0 || m > 0x7fffffffll || n > 0x7fffffffll || k > 0x7fffffffll) {
    set_error("%s: bad extents M=%lld N=%lld K=%lld", what, (long long)m, (long long)n, (long long)k);
    return BT_ERR_ARG;
  }
  return BT_OK;
}

// A operand given as three tensors (bt_gemm_desc.a_split)
struct ASplit {
  int mode;
  const void* A2;
  int64_t lda2, K2, M0, M1;
};
// result given as three tensors side by side along N (bt_gemm_desc.d_split)
struct DSplit {
  void* D1;
  void* D2;
  int64_t ldd1, ldd2, N0, N1;
};

// out[M,N] = T(alpha * (op(A) op(B) + addend))
int plain_gemm(const void* A, bool a_kmajor, int64_t lda, const void* B, bool b_kmajor, int64_t ldb,
               const void* A1, int64_t lda1, const void* B1, int64_t ldb1, int64_t K1, void* D,
               int64_t ldd, int64_t M, int64_t N, int64_t K, int dtype, bool out_fp32,
               const float* addend, int64_t ld_add, const float* alpha, int32_t* status,
               cudaStream_t s, const void* addend_t = nullptr, int64_t ld_add_t = 0,
               const ASplit* split = nullptr, const DSplit* dsplit = nullptr) {
  Launch L;
  L.dtype = dtype;
  out_fp32 = out_fp32 || dtype == BT_FP32;
  L.a0 = operand(A, a_kmajor, M, K, lda);
  L.b0 = operand(B, b_kmajor, N, K, ldb);
  if (split != nullptr && split->mode == gemm::A_SPLIT_K) {
    // A = [A | A1 | A2] along K, one B spanning the whole contraction
    L.a_split = gemm::A_SPLIT_K;
    L.a1 = operand(A1, a_kmajor, M, K1, lda1);
    L.a2 = operand(split->A2, a_kmajor, M, split->K2, split->lda2);
    L.b0 = operand(B, b_kmajor, N, K + K1 + split->K2, ldb);
  } else if (split != nullptr && split->mode == gemm::A_SPLIT_M) {
    // the rows of op(A) are three tensors stacked along M
    L.a_split = gemm::A_SPLIT_M;
    L.a0 = operand(A, a_kmajor, split->M0, K, lda);
    L.a1 = operand(A1, a_kmajor, split->M1, K, lda1);
    L.a2 = operand(split->A2, a_kmajor, M - split->M0 - split->M1, K, split->lda2);
  } else if (A1 != nullptr) {
    L.two_pairs = true;
    L.a1 = operand(A1, a_kmajor, M, K1, lda1);
    L.b1 = operand(B1, b_kmajor, N, K1, ldb1);
  }
  L.p.M = static_cast<int>(M);
  L.p.N = static_cast<int>(N);
  L.p.status = status;
  L.p.out = D;
  L.p.ldo = ldd;
  L.p.out_fp32 = out_fp32 ? 1 : 0;
  L.p.addend = addend;
  L.p.ld_add = ld_add;
  L.p.alpha = alpha;
  L.p.addend_t = addend_t;
  L.p.ld_add_t = ld_add_t;
  L.p.vec_ok = rows_aligned(D, ldd, out_fp32 ? 4 : 2) && rows_aligned(addend, ld_add, 4) &&
               rows_aligned(addend_t, ld_add_t, esize(dtype));
  if (dsplit != nullptr) {
    L.p.out1 = dsplit->D1;
    L.p.out2 = dsplit->D2;
    L.p.ldo1 = dsplit->ldd1;
    L.p.ldo2 = dsplit->ldd2;
    L.p.n_seg0 = static_cast<int>(dsplit->N0);
    L.p.n_seg1 = static_cast<int>(dsplit->N1);
    L.p.vec_ok = L.p.vec_ok && rows_aligned(dsplit->D1, dsplit->ldd1, out_fp32 ? 4 : 2) &&
                 rows_aligned(dsplit->D2, dsplit->ldd2, out_fp32 ? 4 : 2);
  }
  return gemm::launch<gemm::EPI_PLAIN>(L, s);
}

}  // namespace
}  // namespace bt

extern "C" int bt_set_gemm_cta_pairs(int enable) {
  const int prev = bt::gemm::pair_mode();
  if (enable >= 0) bt::gemm::pair_mode() = enable ? 1 : 0;
  return prev;
}

// the tensor-core kernels' copy of the wait limit (called by bt_set_wait_limit_ms in rmsnorm.cu)
int bt_internal_set_wait_limit_tc(unsigned long long ns) {
  return bt::ptx::set_wait_limit_ns(ns) == cudaSuccess ? 0 : -1;
}

extern "C" int bt_set_gemm_group_rows(int row_tiles) {
  const int prev = bt::gemm::group_m_override();
  if (row_tiles >= 0) bt::gemm::group_m_override() = row_tiles;
  return prev;
}

extern "C" int bt_set_gemm_tile_stores(int enable) {
  const int prev = bt::gemm::tma_out_mode();
  if (enable >= 0) bt::gemm::tma_out_mode() = enable ? 1 : 0;
  return prev;
}

extern "C" int bt_set_gemm_dynamic_tiles(int enable) {
  const int prev = bt::gemm::dynamic_tiles();
  if (enable >= 0) bt::gemm::dynamic_tiles() = enable ? 1 : 0;
  return prev;
}

extern "C" int bt_gemm(const void* A, const void* B, void* D, int64_t M, int64_t N, int64_t K,
                       int64_t lda, int64_t ldb, int64_t ldd, int a_kmajor, int b_kmajor,
                       int in_dtype, int out_dtype, const float* addend, int64_t ld_addend,
                       const float* alpha, int32_t* status, void* stream) {
  using namespace bt;
  BT_CHECK_ARG(is_tc(in_dtype), "gemm: operands must be bf16, fp16 or fp32 (got dtype %d)", in_dtype);
  BT_CHECK_ARG(out_dtype == in_dtype || out_dtype == BT_FP32,
               "gemm: result must have the operand dtype or be fp32");
  BT_CHECK_ARG(A && B && D, "gemm: null pointer");
  if (int rc = check_dims("gemm", M, N, K)) return rc;
  BT_CHECK_ARG(ldd >= N && (addend == nullptr || ld_addend >= N), "gemm: result stride too small");
  return plain_gemm(A, a_kmajor != 0, lda, B, b_kmajor != 0, ldb, nullptr, 0, nullptr, 0, 0, D, ldd,
                    M, N, K, in_dtype, out_dtype == BT_FP32, addend, ld_addend, alpha,
                    status, static_cast<cudaStream_t>(stream));
}

extern "C" int bt_gemm_ex(const bt_gemm_desc* d, int32_t* status, void* stream) {
  using namespace bt;
  BT_CHECK_ARG(d != nullptr, "gemm_ex: null descriptor");
  BT_CHECK_ARG(is_tc(d->in_dtype), "gemm_ex: operands must be bf16, fp16 or fp32 (got dtype %d)",
               d->in_dtype);
  BT_CHECK_ARG(d->out_dtype == d->in_dtype || d->out_dtype == BT_FP32,
               "gemm_ex: result must have the operand dtype or be fp32");
  BT_CHECK_ARG(d->A && d->B && d->D, "gemm_ex: null pointer");
  if (int rc = check_dims("gemm_ex", d->M, d->N, d->K)) return rc;
  BT_CHECK_ARG(d->a_split >= 0 && d->a_split <= 2, "gemm_ex: a_split must be 0, 1 or 2");
  ASplit split{d->a_split, d->A2, d->lda2, d->K2, d->M0, d->M1};
  if (d->a_split != 0) {
    BT_CHECK_ARG(d->A1 != nullptr && d->A2 != nullptr && d->B1 == nullptr,
                 "gemm_ex: a split A operand needs A, A1 and A2 and takes no B1");
    if (d->a_split == 1) {
      if (int rc = check_dims("gemm_ex (K-split)", d->M, d->K1, d->K2)) return rc;
    } else {
      BT_CHECK_ARG(d->M0 > 0 && d->M1 > 0 && d->M0 + d->M1 < d->M, "gemm_ex: M-split needs 0 < M0, M1 and M0 + M1 < M");
    }
  }
  DSplit dsplit{d->D1, d->D2, d->ldd1, d->ldd2, d->N0, d->N1};
  if (d->d_split != 0) {
    BT_CHECK_ARG(d->D1 != nullptr && d->D2 != nullptr && d->addend == nullptr && d->addend_t == nullptr,
                 "gemm_ex: a split result needs D, D1 and D2 and takes no addend");
    BT_CHECK_ARG(d->N0 > 0 && d->N1 > 0 && d->N0 + d->N1 < d->N && d->N0 % 256 == 0 && d->N1 % 256 == 0,
                 "gemm_ex: split result needs 0 < N0, N1 in multiples of 256 with N0 + N1 < N");
    BT_CHECK_ARG(d->ldd >= d->N0 && d->ldd1 >= d->N1 && d->ldd2 >= d->N - d->N0 - d->N1,
                 "gemm_ex: split result stride too small");
  }
  const bool second = d->A1 != nullptr;
  if (second && d->a_split == 0) {
    BT_CHECK_ARG(d->B1 != nullptr, "gemm_ex: second product has A1 but no B1");
    if (int rc = check_dims("gemm_ex (second product)", d->M, d->N, d->K1)) return rc;
  }
  BT_CHECK_ARG((d->d_split != 0 || d->ldd >= d->N) && (d->addend == nullptr || d->ld_addend >= d->N) &&
                   (d->addend_t == nullptr || d->ld_addend_t >= d->N),
               "gemm_ex: result / addend stride too small");
  return plain_gemm(d->A, d->a_kmajor != 0, d->lda, d->B, d->b_kmajor != 0, d->ldb,
                    second ? d->A1 : nullptr, d->lda1, second ? d->B1 : nullptr, d->ldb1,
                    second ? d->K1 : 0, d->D, d->ldd, d->M, d->N, d->K, d->in_dtype,
                    d->out_dtype == BT_FP32, d->addend, d->ld_addend, d->alpha, status,
                    static_cast<cudaStream_t>(stream), d->addend_t, d->ld_addend_t,
                    d->a_split != 0 ? &split : nullptr, d->d_split != 0 ? &dsplit : nullptr);
}

extern "C" int bt_mlp_fwd(const void* x, const void* wg, const void* wu, const void* wd, void* gate,
                          void* up, void* h, void* y, int64_t T, int64_t H, int64_t I, int64_t ld_x,
                          const void* residual, int64_t ld_residual, int dtype, int32_t* status,
                          void* stream) {
  using namespace bt;
  BT_CHECK_ARG(is_tc(dtype), "mlp_fwd: unknown dtype %d", dtype);
  BT_CHECK_ARG(T >= 0, "mlp_fwd: negative T");
  if (T == 0) return BT_OK;
  BT_CHECK_ARG(x && wg && wu && wd && gate && up && h && y, "mlp_fwd: null pointer");
  if (int rc = check_dims("mlp_fwd", T, I, H)) return rc;
  BT_CHECK_ARG(residual == nullptr || ld_residual >= H, "mlp_fwd: residual row stride smaller than H");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int bf16 = dtype;  // operand storage, passed through to the launches
  const int es = esize(dtype);
  {
    // gate | up = x [Wg ; Wu]^T with the SwiGLU epilogue
    gemm::Launch L;
    L.dtype = dtype;
    L.dual_b = true;
    L.a0 = operand(x, true, T, H, ld_x);
    L.b0 = operand(wg, true, I, H, H);
    L.b1 = operand(wu, true, I, H, H);
    L.p.M = static_cast<int>(T);
    L.p.N = static_cast<int>(I);
    L.p.status = status;
    L.p.gate = gate;
    L.p.up = up;
    L.p.h = h;
    L.p.ld_act = I;
    L.p.vec_ok = rows_aligned(gate, I, es) && rows_aligned(up, I, es) && rows_aligned(h, I, es);
    if (int rc = gemm::launch<gemm::EPI_SWIGLU_FWD>(L, s)) return rc;
  }
  // y = h Wd^T (+ residual)
  return plain_gemm(h, true, I, wd, true, I, nullptr, 0, nullptr, 0, 0, y, H, T, H, I, bf16, false,
                    nullptr, 0, nullptr, status, s, residual, ld_residual);
}

extern "C" int bt_mlp_bwd(const void* dy, const void* x, const void* wg, const void* wu,
                          const void* wd, const void* gate, const void* up, const void* h,
                          void* dgate, void* dup, void* dx, void* dwg, void* dwu, void* dwd,
                          int64_t T, int64_t H, int64_t I, int64_t ld_x, int64_t ld_dy,
                          int64_t ld_dgate, int dtype, int32_t* status, void* stream) {
  using namespace bt;
  BT_CHECK_ARG(is_tc(dtype), "mlp_bwd: unknown dtype %d", dtype);
  BT_CHECK_ARG(T > 0, "mlp_bwd: T must be positive");
  BT_CHECK_ARG(dy && x && wg && wu && wd && gate && up && h && dgate && dup, "mlp_bwd: null pointer");
  if (int rc = check_dims("mlp_bwd", T, I, H)) return rc;
  BT_CHECK_ARG(ld_dgate >= I, "mlp_bwd: dgate/dup row stride smaller than I");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int bf16 = dtype;  // operand storage, passed through to the launches
  const int es = esize(dtype);
  {
    // dh = dy Wd (Wd stored [H, I] = [K, N]); epilogue -> dgate, dup
    gemm::Launch L;
    L.dtype = dtype;
    L.a0 = operand(dy, true, T, H, ld_dy);
    L.b0 = operand(wd, false, I, H, I);
    L.p.M = static_cast<int>(T);
    L.p.N = static_cast<int>(I);
    L.p.status = status;
    L.p.gate = const_cast<void*>(gate);
    L.p.up = const_cast<void*>(up);
    L.p.out = dgate;
    L.p.h = dup;
    L.p.ld_act = I;
    L.p.ldo = ld_dgate;
    L.p.vec_ok = rows_aligned(gate, I, es) && rows_aligned(up, I, es) &&
                 rows_aligned(dgate, ld_dgate, es) && rows_aligned(dup, ld_dgate, es);
    if (int rc = gemm::launch<gemm::EPI_SWIGLU_BWD>(L, s)) return rc;
  }
  if (dwd != nullptr) {  // dWd[H, I] = dy^T h
    if (int rc = plain_gemm(dy, false, ld_dy, h, false, I, nullptr, 0, nullptr, 0, 0, dwd, I, H, I, T,
                            bf16, false, nullptr, 0, nullptr, status, s))
      return rc;
  }
  // dgate | dup side by side in one [T, 2I] buffer and dWg | dWu stacked in one [2I, H] buffer:
  // the two weight gradients are one product [dgate | dup]^T x (twice the tiles per launch,
  // so the last wave of tiles is fuller).
  const bool stacked = dwg != nullptr && dwu != nullptr && ld_dgate == 2 * I &&
                       static_cast<const char*>(dup) == static_cast<const char*>(dgate) + I * es &&
                       static_cast<const char*>(dwu) == static_cast<const char*>(dwg) + I * H * es;
  if (stacked) {
    if (int rc = plain_gemm(dgate, false, ld_dgate, x, false, ld_x, nullptr, 0, nullptr, 0, 0, dwg, H,
                            2 * I, H, T, bf16, false, nullptr, 0, nullptr, status, s))
      return rc;
  } else {
    if (dwg != nullptr) {  // dWg[I, H] = dgate^T x
      if (int rc = plain_gemm(dgate, false, ld_dgate, x, false, ld_x, nullptr, 0, nullptr, 0, 0, dwg,
                              H, I, H, T, bf16, false, nullptr, 0, nullptr, status, s))
        return rc;
    }
    if (dwu != nullptr) {  // dWu[I, H] = dup^T x
      if (int rc = plain_gemm(dup, false, ld_dgate, x, false, ld_x, nullptr, 0, nullptr, 0, 0, dwu, H,
                              I, H, T, bf16, false, nullptr, 0, nullptr, status, s))
        return rc;
    }
  }
  if (dx != nullptr) {  // dx[T, H] = dgate Wg + dup Wu  (one accumulator, two K ranges)
    if (int rc = plain_gemm(dgate, true, ld_dgate, wg, false, H, dup, ld_dgate, wu, H, I, dx, H, T, H,
                            I, bf16, false, nullptr, 0, nullptr, status, s))
      return rc;
  }
  return BT_OK;
}

// Two statistics entries per 256-column tile (one per 128-column half).
extern "C" int64_t bt_lce_num_vtiles(int64_t V) {
  return 2 * ((V + bt::gemm::BN - 1) / bt::gemm::BN);
}

extern "C" int bt_lce_logits_stats(const void* hidden, const void* W, const int64_t* labels,
                                   void* logits, float* tile_stats, float* tgt_logit, int64_t rows,
                                   int64_t H, int64_t V, int64_t ld_hidden, int64_t ld_logits,
                                   int64_t v_offset, int64_t ignore_index, int dtype,
                                   int32_t* status, void* stream) {
  using namespace bt;
  BT_CHECK_ARG(is_tc(dtype), "lce_logits_stats: unknown dtype %d", dtype);
  BT_CHECK_ARG(rows >= 0, "lce_logits_stats: negative rows");
  if (rows == 0) return BT_OK;
  BT_CHECK_ARG(hidden && W && labels && logits && tile_stats && tgt_logit,
               "lce_logits_stats: null pointer");
  if (int rc = check_dims("lce_logits_stats", rows, V, H)) return rc;
  BT_CHECK_ARG(ld_logits >= V, "lce_logits_stats: logits stride smaller than V");
  gemm::Launch L;
  L.dtype = dtype;
  L.a0 = operand(hidden, true, rows, H, ld_hidden);
  L.b0 = operand(W, true, V, H, H);
  L.p.M = static_cast<int>(rows);
  L.p.N = static_cast<int>(V);
  L.p.status = status;
  L.p.out = logits;
  L.p.ldo = ld_logits;
  L.p.labels = labels;
  L.p.tile_stats = tile_stats;
  L.p.tgt_logit = tgt_logit;
  L.p.v_offset = v_offset;
  L.p.ignore_index = ignore_index;
  L.p.n_vtiles = static_cast<int>(bt_lce_num_vtiles(V));
  L.p.vec_ok = rows_aligned(logits, ld_logits, esize(dtype));
  return gemm::launch<gemm::EPI_LCE>(L, static_cast<cudaStream_t>(stream));
}

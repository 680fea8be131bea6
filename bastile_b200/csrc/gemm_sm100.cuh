// Persistent, warp-specialised tcgen05 GEMM for sm_100a with pluggable epilogues.
//
//   CTA tile 128 x 256 x 64 (16-bit operands), one CTA per SM, 320 threads:
//     warp 0      TMA producer   - one lane issues the tile loads of a 4-stage ring
//     warp 1      MMA issuer     - owns the 512 TMEM columns, one lane issues tcgen05.mma
//     warps 2..9  epilogue       - two per 32-lane quarter of TMEM, half of the columns each
//   The fp32 accumulator (128 lanes x 256 columns) is double-buffered in tensor
//   memory, so the epilogue of tile i overlaps the main loop of tile i+1.
//
//   Operands may be K-major (rows = M/N index, K contiguous) or MN-major (rows = K
//   index, M/N contiguous); both land in shared memory as 128-byte rows with the
//   128-byte TMA swizzle, which is what the UMMA shared-memory descriptors expect.
//   Ragged M / N / K need no special casing in the main loop: TMA zero-fills reads
//   outside the tensor, and the epilogues bound-check their global accesses.
//
//   Optional main-loop modes
//     dual_b    : the B tile is 128 rows of B0 followed by 128 rows of B1 (same A),
//                 i.e. accumulator columns [0,128) = A*B0^T, [128,256) = A*B1^T;
//     two pairs : the K loop runs over (A0,B0) and then (A1,B1) into one accumulator.
//
//   Two kernels share the epilogues.  gemm_kernel is the layout above.  gemm_kernel_pair
//   (the default) runs 2-CTA clusters on 256 x 256 tiles with tcgen05.mma.cta_group::2:
//   each CTA stages its own 128 rows of A and 128 columns of B (6-stage ring of 32 KB),
//   the leader CTA's warp 1 issues the MMAs for both, tcgen05.commit arrives on both
//   CTAs' barriers, and an eleventh warp (352 threads) issues the B loads next to warp
//   0's A loads.  Tile loads are plain per-CTA TMA loads; nothing is multicast.
//
//   fp32 operands are multiplied as tf32 (K depth 32 per 128-byte row); Geo<T> carries
//   the per-type tile geometry at compile time.
//
//   The plain epilogue can add an fp32 matrix and/or a matrix in the operand type (a
//   residual stream) to the accumulator before the single rounding.
//
//   Every mbarrier wait is bounded (sm100_ptx.cuh); a wait that runs out sets the
//   caller's status word, makes all roles leave their loops, and the CTA still
//   frees its tensor memory before exiting.
#pragma once

#include <atomic>
#include <mutex>

#include "bt_common.cuh"
#include "sm100_ptx.cuh"

namespace bt {
namespace gemm {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;       // k-block in 16-bit elements; every k-block is 128 bytes of K per row
constexpr int kRowBytes = 128;
constexpr int kStages = 4;
constexpr int kEpiWarps = 8;  // two warps per 32-lane TMEM quarter, each takes half of the columns
constexpr int kThreads = 64 + 32 * kEpiWarps;
constexpr int kABytes = BM * BK * 2;
constexpr int kBBytes = BN * BK * 2;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kTmemCols = 512;
constexpr int kGroupM = 16;  // tile rasterisation: walk 16 row-tiles per column-tile
// Result staging for tile stores: every epilogue warp owns two 2 KB buffers (32 rows x 64 bytes,
// 64-byte swizzle) that it fills from registers and hands to cp.async.bulk.tensor stores.
constexpr int kStageOutBytes = 2048;
constexpr int kOutBytes = kEpiWarps * 2 * kStageOutBytes;  // 32 KB
constexpr int kCtrlBytes = 1024;                            // barriers, TMEM slot, abort flag
constexpr int kSmemBytes = kStages * kStageBytes + kCtrlBytes + kOutBytes + 1024 /*alignment slack*/;

// Tile geometry that depends on the operand element size (all rows are 128 bytes).
template <typename T>
struct Geo {
  static constexpr int kBk = kRowBytes / static_cast<int>(sizeof(T));     // K elements per k-block
  static constexpr int kMnBox = kRowBytes / static_cast<int>(sizeof(T));  // M/N elements per MN-major box row
  static constexpr int kBoxBytes = kBk * kRowBytes;                       // one MN-major box
};

enum : int { EPI_PLAIN = 0, EPI_SWIGLU_FWD = 1, EPI_SWIGLU_BWD = 2, EPI_LCE = 3 };

// Status-word bits set when a bounded wait runs out.
enum : int { ST_PRODUCER = 1, ST_MMA_ACC = 2, ST_MMA_FULL = 4, ST_EPILOGUE = 8 };

// How the A operand is assembled from up to three tensors (one B tensor in both cases).
enum : int { A_WHOLE = 0, A_SPLIT_K = 1, A_SPLIT_M = 2 };

struct Params {
  int M, N;        // output extent; with dual_b, N is the width of ONE of the two outputs
  int K0, K1;      // contraction lengths of pair 0 and pair 1 (K1 = 0: single pair)
  int K2;          // A_SPLIT_K: contraction length of the third A tensor (B spans K0 + K1 + K2)
  int a_split;     // A_WHOLE, A_SPLIT_K or A_SPLIT_M
  int m_seg0, m_seg1;  // A_SPLIT_M: rows [0, m_seg0) come from A0, the next m_seg1 from A1, the rest from A2
  int tiles_m, tiles_n, num_tiles;
  int group_m;     // rasterisation: row-tiles walked per column-tile before moving on
  int a_kmajor, b_kmajor, dual_b;
  uint32_t idesc;
  uint64_t a_desc_hi, b_desc_hi;
  uint32_t a_kstep, b_kstep;  // descriptor address step per MMA K slice, 16-byte units
  int32_t* status;
  // Dynamic tile hand-out (pair kernel, optional): word 0 is the next-tile counter, then
  // kSchedRing published tile ids per CTA pair.  nullptr: tiles are dealt round-robin.
  unsigned long long* sched;
  // --- plain epilogue: out = T(alpha * (acc + addend))
  void* out;
  int64_t ldo;
  // plain epilogue, result split along N over three tensors (n_seg0 > 0): columns [0, n_seg0) go
  // to out, the next n_seg1 to out1, the rest to out2; segment widths are whole tiles
  void* out1;
  void* out2;
  int64_t ldo1, ldo2;
  int n_seg0, n_seg1;
  int out_fp32;
  int vec_ok;  // rows of every global tensor the epilogue touches are 16-byte aligned
  int tma_out; // 16-bit results leave through shared memory and tile stores (tensor maps tmO0..2)
  const float* addend;
  int64_t ld_add;
  const void* addend_t;  // second addend, stored in the operand type (a residual stream)
  int64_t ld_add_t;
  const float* alpha;
  // --- SwiGLU epilogues (row stride ld_act)
  void* gate;  // fwd: out, bwd: in
  void* up;    // fwd: out, bwd: in
  void* h;     // fwd: out (h), bwd: out (dup); bwd writes dgate to `out`
  int64_t ld_act;
  // --- fused cross-entropy epilogue
  const int64_t* labels;
  float* tile_stats;
  float* tgt_logit;
  int64_t v_offset, ignore_index;
  int n_vtiles;
};

__device__ __forceinline__ void tile_coords(const Params& p, int tile, int* m_idx, int* n_idx) {
  const int per_group = p.group_m * p.tiles_n;
  const int g = tile / per_group;
  const int first_m = g * p.group_m;
  const int gs = min(p.tiles_m - first_m, p.group_m);
  const int r = tile - g * per_group;
  *m_idx = first_m + r % gs;
  *n_idx = r / gs;
}

template <typename T>
__device__ __forceinline__ float round_through(float x) {
  return Cvt<T>::to_f(Cvt<T>::from_f(x));
}

// Store 32 consecutive values of one row (vector path when the span is whole and aligned).
__device__ __forceinline__ void store_row32_f32(float* dst, const float (&v)[32], int valid, bool vec);

template <typename T>
__device__ __forceinline__ void store_row32(T* dst, const float (&v)[32], int valid, bool vec) {
  if constexpr (sizeof(T) == 4) {
    store_row32_f32(dst, v, valid, vec);
  } else if (vec && valid >= 32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float f[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = v[i * 8 + e];
      st_once_v4(dst + i * 8, Cvt<T>::pack(f));
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < valid) dst[j] = Cvt<T>::from_f(v[j]);
  }
}
__device__ __forceinline__ void store_row32_f32(float* dst, const float (&v)[32], int valid,
                                                bool vec) {
  if (vec && valid >= 32) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      *reinterpret_cast<float4*>(dst + i * 4) =
          make_float4(v[i * 4], v[i * 4 + 1], v[i * 4 + 2], v[i * 4 + 3]);
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < valid) dst[j] = v[j];
  }
}
template <typename T>
__device__ __forceinline__ void load_row32(const T* src, float (&v)[32], int valid, bool vec) {
  if constexpr (sizeof(T) == 4) {
    if (vec && valid >= 32) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint4 t = ld_once_v4(src + i * 4);
        v[i * 4] = __uint_as_float(t.x);
        v[i * 4 + 1] = __uint_as_float(t.y);
        v[i * 4 + 2] = __uint_as_float(t.z);
        v[i * 4 + 3] = __uint_as_float(t.w);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = (j < valid) ? src[j] : 0.f;
    }
  } else if (vec && valid >= 32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float f[8];
      Cvt<T>::unpack(ld_once_v4(src + i * 8), f);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[i * 8 + e] = f[e];
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = (j < valid) ? Cvt<T>::to_f(src[j]) : 0.f;
  }
}

// A warp's way out for 16-bit results: 32 rows x 32 columns per store.  Each lane writes its row
// (64 bytes) into the warp's staging buffer with the 64-byte swizzle the tensor map expects
// (16-byte piece i of row r lands at piece i ^ ((r >> 1) & 3): conflict-free for the eight lanes
// of a store phase), then one lane issues the tile store.  Two buffers alternate; before a buffer
// is refilled the store that last read it must have finished reading (wait_group.read 1).
// base == 0: the launch stores straight from registers instead.  Must be called by all 32 lanes.
struct OutStage {
  uint32_t base;
  uint32_t count;
};

template <typename T>
__device__ __forceinline__ void stage_store32(OutStage& st, const CUtensorMap* tm,
                                              const float (&v)[32], int col0, int row0, int lane) {
  if constexpr (sizeof(T) == 2) {
    const uint32_t buf = st.base + (st.count & 1u) * kStageOutBytes;
    ++st.count;
    if (lane == 0) ptx::bulk_wait_group_read<1>();
    __syncwarp();
    const uint32_t row = buf + static_cast<uint32_t>(lane) * 64u;
    const uint32_t sw = (static_cast<uint32_t>(lane) >> 1) & 3u;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float f[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = v[i * 8 + e];
      ptx::st_shared_v4(row + ((static_cast<uint32_t>(i) ^ sw) << 4), Cvt<T>::pack(f));
    }
    ptx::fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      ptx::tma_store_2d(tm, buf, col0, row0);
      ptx::bulk_commit_group();
    }
  }
}

// ------------------------------------------------------------------ epilogues
template <typename T>
__device__ __forceinline__ void epi_plain(const Params& p, uint32_t taddr, int64_t row, int n0,
                                          int half, OutStage& stg, const CUtensorMap* tmO0,
                                          const CUtensorMap* tmO1, const CUtensorMap* tmO2, int lane) {
  const float alpha = p.alpha != nullptr ? __ldg(p.alpha) : 1.0f;
  const bool row_ok = row < p.M;
  const int row0 = static_cast<int>(row) - lane;  // first row of this warp's 32
  // where this tile's columns live: one result tensor, or one of three side by side
  void* out = p.out;
  int64_t ldo = p.ldo;
  int col_shift = 0, n_end = p.N;
  const CUtensorMap* tmo = tmO0;
  if (p.n_seg0 > 0) {
    if (n0 < p.n_seg0) {
      n_end = p.n_seg0;
    } else if (n0 < p.n_seg0 + p.n_seg1) {
      out = p.out1;
      ldo = p.ldo1;
      col_shift = p.n_seg0;
      n_end = p.n_seg0 + p.n_seg1;
      tmo = tmO1;
    } else {
      out = p.out2;
      ldo = p.ldo2;
      col_shift = p.n_seg0 + p.n_seg1;
      tmo = tmO2;
    }
  }
#pragma unroll 1
  for (int c = half * (BN / 64); c < (half + 1) * (BN / 64); ++c) {
    float v[32], res[32];
    const int col0 = n0 + c * 32;
    const int valid = n_end - col0;
    const bool add_res = p.addend_t != nullptr && row_ok && valid > 0;
    if (add_res)  // in flight while the accumulator chunk is fetched
      load_row32<T>(static_cast<const T*>(p.addend_t) + row * p.ld_add_t + col0, res, valid,
                    p.vec_ok);
    ptx::tmem_ld_32cols(taddr + c * 32, v);
    if (stg.base != 0) {
      // every lane computes (rows past M hold zeros and are clipped by the store)
      if (valid > 0 && row0 < p.M) {
        if (add_res) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] += res[j];
        }
        if (p.addend != nullptr && row_ok) {
          const float* a = p.addend + row * p.ld_add + col0;
          if (valid >= 32) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float4 t = *reinterpret_cast<const float4*>(a + i * 4);
              v[i * 4] += t.x;
              v[i * 4 + 1] += t.y;
              v[i * 4 + 2] += t.z;
              v[i * 4 + 3] += t.w;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < valid) v[j] += a[j];
          }
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] *= alpha;
        stage_store32<T>(stg, tmo, v, col0 - col_shift, row0, lane);
      }
      continue;
    }
    if (row_ok && valid > 0) {
      if (add_res) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] += res[j];
      }
      if (p.addend != nullptr) {
        const float* a = p.addend + row * p.ld_add + col0;
        if (p.vec_ok && valid >= 32) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float4 t = *reinterpret_cast<const float4*>(a + i * 4);
            v[i * 4] += t.x;
            v[i * 4 + 1] += t.y;
            v[i * 4 + 2] += t.z;
            v[i * 4 + 3] += t.w;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < valid) v[j] += a[j];
        }
      }
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] *= alpha;
      if (p.out_fp32)
        store_row32_f32(static_cast<float*>(out) + row * ldo + (col0 - col_shift), v, valid, p.vec_ok);
      else
        store_row32<T>(static_cast<T*>(out) + row * ldo + (col0 - col_shift), v, valid, p.vec_ok);
    }
  }
}

// Accumulator columns [0,128) = gate, [128,256) = up for output columns n0 .. n0+127.
template <typename T>
__device__ __forceinline__ void epi_swiglu_fwd(const Params& p, uint32_t taddr, int64_t row,
                                               int n0, int half, OutStage& stg,
                                               const CUtensorMap* tm_gate, const CUtensorMap* tm_up,
                                               const CUtensorMap* tm_h, int lane) {
  const bool row_ok = row < p.M;
  const int row0 = static_cast<int>(row) - lane;
#pragma unroll 1
  for (int c = half * (BN / 128); c < (half + 1) * (BN / 128); ++c) {
    float g[32], u[32];
    ptx::tmem_ld_32cols(taddr + c * 32, g);
    ptx::tmem_ld_32cols(taddr + BN / 2 + c * 32, u);
    const int col0 = n0 + c * 32;
    const int valid = p.N - col0;
    if (stg.base != 0) {
      if (valid > 0 && row0 < p.M) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          g[j] = round_through<T>(g[j]);
          u[j] = round_through<T>(u[j]);
        }
        stage_store32<T>(stg, tm_gate, g, col0, row0, lane);
        stage_store32<T>(stg, tm_up, u, col0, row0, lane);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float silu = round_through<T>(g[j] * __fdividef(1.0f, 1.0f + __expf(-g[j])));
          g[j] = silu * u[j];
        }
        stage_store32<T>(stg, tm_h, g, col0, row0, lane);
      }
      continue;
    }
    if (row_ok && valid > 0) {
      float hh[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        g[j] = round_through<T>(g[j]);
        u[j] = round_through<T>(u[j]);
        const float silu = round_through<T>(g[j] * __fdividef(1.0f, 1.0f + __expf(-g[j])));
        hh[j] = silu * u[j];
      }
      const int64_t off = row * p.ld_act + col0;
      store_row32<T>(static_cast<T*>(p.gate) + off, g, valid, p.vec_ok);
      store_row32<T>(static_cast<T*>(p.up) + off, u, valid, p.vec_ok);
      store_row32<T>(static_cast<T*>(p.h) + off, hh, valid, p.vec_ok);
    }
  }
}

// Accumulator = dh tile; reads saved gate/up, writes dgate (p.out) and dup (p.h).
template <typename T>
__device__ __forceinline__ void epi_swiglu_bwd(const Params& p, uint32_t taddr, int64_t row,
                                               int n0, int half, OutStage& stg,
                                               const CUtensorMap* tm_dgate, const CUtensorMap* tm_dup,
                                               int lane) {
  const bool row_ok = row < p.M;
  const int row0 = static_cast<int>(row) - lane;
#pragma unroll 1
  for (int c = half * (BN / 64); c < (half + 1) * (BN / 64); ++c) {
    const int col0 = n0 + c * 32;
    const int valid = p.N - col0;
    const bool live = row_ok && valid > 0;
    const int64_t off = row * p.ld_act + col0;
    float d[32], g[32], u[32];
    if (live) {  // the global loads are in flight while the accumulator chunk is fetched
      load_row32<T>(static_cast<const T*>(p.gate) + off, g, valid, p.vec_ok);
      load_row32<T>(static_cast<const T*>(p.up) + off, u, valid, p.vec_ok);
    }
    ptx::tmem_ld_32cols(taddr + c * 32, d);
    if (stg.base != 0) {
      if (valid > 0 && row0 < p.M) {
        // rows past M (lanes that loaded nothing) hold a zero accumulator: whatever g and u
        // contain there is multiplied by dh = 0 unless it is not finite, and the store clips them
        if (!live) {
#pragma unroll
          for (int j = 0; j < 32; ++j) g[j] = u[j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float dh = round_through<T>(d[j]);
          const float sg = __fdividef(1.0f, 1.0f + __expf(-g[j]));
          d[j] = dh * (sg * (1.0f + g[j] * (1.0f - sg))) * u[j];  // dgate
          g[j] = dh * (g[j] * sg);                                 // dup
        }
        stage_store32<T>(stg, tm_dgate, d, col0, row0, lane);
        stage_store32<T>(stg, tm_dup, g, col0, row0, lane);
      }
      continue;
    }
    if (live) {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float dh = round_through<T>(d[j]);
        // results are rounded to 16 bits: the approximate exp / reciprocal are far inside that
        const float sg = __fdividef(1.0f, 1.0f + __expf(-g[j]));
        d[j] = dh * (sg * (1.0f + g[j] * (1.0f - sg))) * u[j];  // dgate
        g[j] = dh * (g[j] * sg);                                 // dup
      }
      const int64_t off_o = row * p.ldo + col0;  // dgate / dup may live in a wider buffer
      store_row32<T>(static_cast<T*>(p.out) + off_o, d, valid, p.vec_ok);
      store_row32<T>(static_cast<T*>(p.h) + off_o, g, valid, p.vec_ok);
    }
  }
}

// Accumulator = logits tile: per-row (max, sum exp) of the tile, the target logit, and
// the logits themselves rounded to T.
template <typename T>
__device__ __forceinline__ void epi_lce(const Params& p, uint32_t taddr, int64_t row, int n0,
                                        int n_idx, int half, OutStage& stg,
                                        const CUtensorMap* tm_logits, int lane) {
  const bool row_ok = row < p.M;
  const int row0 = static_cast<int>(row) - lane;
  constexpr float kNegBig = -1e30f;
  int tgt_col = -1;  // column of the label inside this tile, if it is here
  bool owned = false;
  if (row_ok) {
    const int64_t label = p.labels[row];
    const int64_t loc = label - p.v_offset;
    owned = (label != p.ignore_index) && loc >= 0 && loc < p.N;
    if (owned && loc >= n0 + half * (BN / 2) && loc < n0 + (half + 1) * (BN / 2))
      tgt_col = static_cast<int>(loc - n0);
  }
  float mx = kNegBig, sum = 0.f, tgt = 0.f;
#pragma unroll 1
  for (int c = half * (BN / 64); c < (half + 1) * (BN / 64); ++c) {
    float v[32];
    ptx::tmem_ld_32cols(taddr + c * 32, v);
    const int col0 = n0 + c * 32;
    const int valid = p.N - col0;
    if (valid > 0) {
      float cmax = kNegBig;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        v[j] = (j < valid) ? round_through<T>(v[j]) : kNegBig;
        cmax = fmaxf(cmax, v[j]);
      }
      const float newm = fmaxf(mx, cmax);
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < 32; ++j) s += __expf(v[j] - newm);
      sum = sum * __expf(mx - newm) + s;
      mx = newm;
      if (tgt_col >= c * 32 && tgt_col < c * 32 + 32) {
        const int jj = tgt_col - c * 32;
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j == jj) tgt = v[j];
      }
      if (stg.base != 0) {
        if (row0 < p.M) stage_store32<T>(stg, tm_logits, v, col0, row0, lane);
      } else if (row_ok) {
        store_row32<T>(static_cast<T*>(p.out) + row * p.ldo + col0, v, valid, p.vec_ok);
      }
    }
  }
  if (row_ok) {
    // one statistics entry per 128 columns (a half tile); an all-padding half stays (-1e30, 0)
    *reinterpret_cast<float2*>(p.tile_stats + (row * p.n_vtiles + n_idx * 2 + half) * 2) =
        make_float2(mx, sum);
    if (tgt_col >= 0)
      p.tgt_logit[row] = tgt;
    else if (n_idx == 0 && half == 0 && !owned)
      p.tgt_logit[row] = 0.f;
  }
}

// Which tensor map, and which coordinates inside it, hold the A tile of rows m0.. for k-block kb.
struct ASource {
  const CUtensorMap* map;
  int k, m;
};
__device__ __forceinline__ ASource a_source(const Params& p, const CUtensorMap* a0,
                                            const CUtensorMap* a1, const CUtensorMap* a2, int kb,
                                            int nkb0, int nkb1, int m0, int kbk) {
  ASource r;
  if (p.a_split == A_SPLIT_M) {
    // the M extent is three tensors stacked (segment lengths are multiples of the tile height)
    r.k = kb * kbk;
    if (m0 < p.m_seg0) {
      r.map = a0;
      r.m = m0;
    } else if (m0 < p.m_seg0 + p.m_seg1) {
      r.map = a1;
      r.m = m0 - p.m_seg0;
    } else {
      r.map = a2;
      r.m = m0 - p.m_seg0 - p.m_seg1;
    }
    return r;
  }
  // the K extent is one tensor, two operand pairs (A_WHOLE with K1 > 0) or three A tensors side
  // by side against one B tensor (A_SPLIT_K; K0 and K1 are whole numbers of k-blocks)
  r.m = m0;
  if (kb < nkb0) {
    r.map = a0;
    r.k = kb * kbk;
  } else if (kb < nkb0 + nkb1) {
    r.map = a1;
    r.k = (kb - nkb0) * kbk;
  } else {
    r.map = a2;
    r.k = (kb - nkb0 - nkb1) * kbk;
  }
  return r;
}

// --------------------------------------------------------------------- kernel
template <int EPI, typename T>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmB0,
            const __grid_constant__ CUtensorMap tmA1, const __grid_constant__ CUtensorMap tmB1,
            const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmO0,
            const __grid_constant__ CUtensorMap tmO1, const __grid_constant__ CUtensorMap tmO2,
            const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* empty = full + kStages;
  uint64_t* tfull = empty + kStages;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      ptx::mbar_init(&full[i], 1);
      ptx::mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&tfull[i], 1);
      ptx::mbar_init(&tempty[i], 32 * kEpiWarps);
    }
    *cta_abort = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tmA0);
    ptx::prefetch_tensormap(&tmB0);
    if ((p.K1 > 0 && p.a_split == A_WHOLE) || p.dual_b) ptx::prefetch_tensormap(&tmB1);
    if (p.K1 > 0 || p.a_split != A_WHOLE) ptx::prefetch_tensormap(&tmA1);
    if (p.a_split != A_WHOLE) ptx::prefetch_tensormap(&tmA2);
    if (p.tma_out) ptx::prefetch_tensormap(&tmO0);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, kTmemCols);
    ptx::tmem_relinquish_alloc_permit();
  }
  ptx::tcgen05_fence_before_sync();
  __syncthreads();
  ptx::tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  grid_dependency_wait();  // barriers, tensor memory and descriptors were set up while the previous kernel drained

  constexpr int kBk = Geo<T>::kBk, kMnBox = Geo<T>::kMnBox, kBoxBytes = Geo<T>::kBoxBytes;
  const int nkb0 = (p.K0 + kBk - 1) / kBk;
  const int nkb1 = (p.K1 + kBk - 1) / kBk;
  const int nkb = nkb0 + nkb1 + (p.K2 + kBk - 1) / kBk;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
        int m_idx, n_idx;
        tile_coords(p, tile, &m_idx, &n_idx);
        const int m0 = m_idx * BM;
        const int n0 = n_idx * (p.dual_b ? BN / 2 : BN);
        for (int kb = 0; kb < nkb; ++kb) {
          if (!ptx::mbar_wait(&empty[stage], phase ^ 1u, cta_abort, p.status, ST_PRODUCER)) {
            ok = false;
            break;
          }
          ptx::mbar_arrive_expect_tx(&full[stage], kStageBytes);
          const ASource as = a_source(p, &tmA0, &tmA1, &tmA2, kb, nkb0, nkb1, m0, kBk);
          const bool second = p.a_split == A_WHOLE && kb >= nkb0;
          const int kb_b = second ? (kb - nkb0) * kBk : kb * kBk;  // A_SPLIT_K: B's K range runs on
          const CUtensorMap* ta = as.map;
          const CUtensorMap* tb = second ? &tmB1 : &tmB0;
          uint8_t* sa = smem + stage * kStageBytes;
          uint8_t* sb = sa + kABytes;
          if (p.a_kmajor) {
            ptx::tma_load_2d(sa, ta, as.k, as.m, &full[stage]);
          } else {
#pragma unroll
            for (int j = 0; j < BM / kMnBox; ++j)
              ptx::tma_load_2d(sa + j * kBoxBytes, ta, as.m + j * kMnBox, as.k, &full[stage]);
          }
          if (p.dual_b) {
            ptx::tma_load_2d(sb, &tmB0, kb_b, n0, &full[stage]);
            ptx::tma_load_2d(sb + kBBytes / 2, &tmB1, kb_b, n0, &full[stage]);
          } else if (p.b_kmajor) {
            ptx::tma_load_2d(sb, tb, kb_b, n0, &full[stage]);
          } else {
#pragma unroll
            for (int j = 0; j < BN / kMnBox; ++j)
              ptx::tma_load_2d(sb + j * kBoxBytes, tb, n0 + j * kMnBox, kb_b, &full[stage]);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok || *cta_abort != 0) {
        // Something gave up: give the copies that are still in flight time to land
        // before this CTA's shared memory can be handed to another CTA.
        const uint64_t t0 = ptx::globaltimer_ns();
        while (ptx::globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
        if (!ptx::mbar_wait(&tempty[acc], acc_phase ^ 1u, cta_abort, p.status, ST_MMA_ACC)) break;
        ptx::tcgen05_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < nkb; ++kb) {
          if (!ptx::mbar_wait(&full[stage], phase, cta_abort, p.status, ST_MMA_FULL)) {
            ok = false;
            break;
          }
          ptx::tcgen05_fence_after_sync();
          const uint32_t a_addr = ptx::smem_u32(smem + stage * kStageBytes);
          const uint64_t a_desc = ptx::smem_desc(p.a_desc_hi, a_addr);
          const uint64_t b_desc = ptx::smem_desc(p.b_desc_hi, a_addr + kABytes);
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {  // 4 K slices of 32 bytes per k-block
            if constexpr (sizeof(T) == 4)
              ptx::umma_tf32(d_tmem, a_desc + static_cast<uint64_t>(kk * p.a_kstep),
                             b_desc + static_cast<uint64_t>(kk * p.b_kstep), p.idesc,
                             (kb | kk) != 0 ? 1u : 0u);
            else
              ptx::umma_f16(d_tmem, a_desc + static_cast<uint64_t>(kk * p.a_kstep),
                            b_desc + static_cast<uint64_t>(kk * p.b_kstep), p.idesc,
                            (kb | kk) != 0 ? 1u : 0u);
          }
          ptx::umma_commit(&empty[stage]);  // frees the smem stage when these MMAs retire
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        ptx::umma_commit(&tfull[acc]);  // accumulator complete -> epilogue
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
    const int half = (warp - 2) >> 2;  // which half of the accumulator columns
    int acc = 0;
    uint32_t acc_phase = 0;
    OutStage stg;
    stg.base = p.tma_out ? ptx::smem_u32(smem + kStages * kStageBytes + kCtrlBytes) +
                               static_cast<uint32_t>(warp - 2) * (2 * kStageOutBytes)
                         : 0u;
    stg.count = 0;
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
      int m_idx, n_idx;
      tile_coords(p, tile, &m_idx, &n_idx);
      // all 32 lanes leave together: what follows is warp-synchronous (tcgen05.ld.sync.aligned)
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(&tfull[acc], acc_phase, cta_abort, p.status, ST_EPILOGUE)))
        break;
      ptx::tcgen05_fence_after_sync();
      const uint32_t taddr =
          tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BN);
      const int64_t row = static_cast<int64_t>(m_idx) * BM + quarter * 32 + lane;
      if (EPI == EPI_PLAIN) epi_plain<T>(p, taddr, row, n_idx * BN, half, stg, &tmO0, &tmO1, &tmO2, lane);
      if (EPI == EPI_SWIGLU_FWD)
        epi_swiglu_fwd<T>(p, taddr, row, n_idx * (BN / 2), half, stg, &tmO0, &tmO1, &tmO2, lane);
      if (EPI == EPI_SWIGLU_BWD) epi_swiglu_bwd<T>(p, taddr, row, n_idx * BN, half, stg, &tmO0, &tmO1, lane);
      if (EPI == EPI_LCE) epi_lce<T>(p, taddr, row, n_idx * BN, n_idx, half, stg, &tmO0, lane);
      ptx::tcgen05_fence_before_sync();
      ptx::mbar_arrive(&tempty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    // this warp's tile stores must have left shared memory (and landed) before the CTA goes away
    if (stg.base != 0 && lane == 0) ptx::bulk_wait_group<0>();
  }

  // ------------------------------------------------------------------ teardown
  ptx::tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tcgen05_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------- kernel, CTA pairs
// Same roles and epilogues, but two CTAs of a 2-CTA cluster work on one 256 x 256 tile with
// tcgen05.mma.cta_group::2: each CTA stages its own 128 rows of A and its own 128 columns
// of B (32 KB per stage instead of 48 KB, so the ring is 6 deep), the leader CTA's MMA lane
// issues for both, and each CTA's epilogue drains its own 128 accumulator rows.
//   full[s]    lives in the leader: armed by the leader's producer with the bytes of BOTH
//              CTAs; each CTA's tile loads credit it (plain loads, no multicast).
//   empty[s], tfull[a]  live in both CTAs; the leader's commit arrives on both copies.
//   tempty[a]  lives in the leader; epilogue threads of both CTAs arrive on it.
constexpr int kStages2 = 6;
constexpr int kPairProducerB = 2 + kEpiWarps;       // warp index of the second producer
constexpr int kThreadsPair = kThreads + 32;
constexpr int kStageBytes2 = kABytes + kBBytes / 2;
constexpr int kSmemBytes2 = kStages2 * kStageBytes2 + kCtrlBytes + kOutBytes + 1024;

// ---- dynamic tile hand-out -------------------------------------------------------------
// With a fixed round-robin deal a CTA pair that gets its SMs late (a collective's kernel is
// sitting on them when the GEMM starts) still has its whole share of tiles in front of it and
// the launch takes up to twice as long.  In dynamic mode the leader CTA's A-producer draws
// tile numbers from a global counter, one tile ahead of the one it is loading, and publishes
// them in a small ring in global memory; every other role of the pair - the second
// producer, the peer CTA's producers, the MMA issuer, the epilogue warps - reads its i-th
// tile from ring slot i % kSchedRing (tag i + 1 in the upper half says the slot is fresh).
// How far the drawing thread can be ahead of the slowest reader: one tile published in
// advance, up to kStages2 tiles of loads in flight when a tile is a single k-block, and two
// accumulators between the MMA issuer and the epilogue - nine tiles, so sixteen slots never
// wrap onto an unread entry.  The host clears counter and ring before the launch.
constexpr int kSchedRing = 16;
constexpr int kSchedMaxPairs = 256;
constexpr int kSchedWords = 1 + kSchedMaxPairs * kSchedRing;
constexpr int kSchedSlots = 32;
__device__ unsigned long long g_tile_sched[kSchedSlots][kSchedWords];

__device__ __forceinline__ int sched_draw(const Params& p) {
  const unsigned int t = atomicAdd(reinterpret_cast<unsigned int*>(p.sched), 1u);
  return t < static_cast<unsigned int>(p.num_tiles) ? static_cast<int>(t) : -1;
}
__device__ __forceinline__ void sched_publish(const Params& p, int pair, int i, int tile) {
  unsigned long long* slot = p.sched + 1 + pair * kSchedRing + (i % kSchedRing);
  const unsigned long long v = (static_cast<unsigned long long>(i + 1) << 32) |
                               static_cast<unsigned int>(tile + 1);
  asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(slot), "l"(v) : "memory");
}
// The i-th tile of this pair (-1: no more tiles, or the wait was given up).
__device__ __forceinline__ int sched_wait(const Params& p, int pair, int npairs, int i,
                                          volatile int* cta_abort, int status_bit) {
  if (p.sched == nullptr) {
    const int t = pair + i * npairs;
    return t < p.num_tiles ? t : -1;
  }
  const unsigned long long* slot = p.sched + 1 + pair * kSchedRing + (i % kSchedRing);
  const uint64_t t0 = ptx::globaltimer_ns();
  for (;;) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(slot) : "memory");
    if (static_cast<unsigned int>(v >> 32) == static_cast<unsigned int>(i + 1))
      return static_cast<int>(static_cast<unsigned int>(v)) - 1;
    if (*cta_abort != 0) return -1;
    if (ptx::globaltimer_ns() - t0 > *reinterpret_cast<volatile unsigned long long*>(&ptx::g_wait_limit_ns)) {
      *cta_abort = 1;
      if (p.status != nullptr) atomicOr(p.status, status_bit);
      return -1;
    }
    __nanosleep(200);
  }
}

template <int EPI, typename T>
__global__ void __launch_bounds__(kThreadsPair, 1)
gemm_kernel_pair(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmB0,
                 const __grid_constant__ CUtensorMap tmA1, const __grid_constant__ CUtensorMap tmB1,
                 const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmO0,
            const __grid_constant__ CUtensorMap tmO1, const __grid_constant__ CUtensorMap tmO2,
            const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages2 * kStageBytes2);
  uint64_t* empty = full + kStages2;
  uint64_t* tfull = empty + kStages2;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();  // 0 = leader
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages2; ++i) {
      ptx::mbar_init(&full[i], 1);
      ptx::mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&tfull[i], 1);
      ptx::mbar_init(&tempty[i], 2 * 32 * kEpiWarps);
    }
    *cta_abort = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tmA0);
    ptx::prefetch_tensormap(&tmB0);
    if ((p.K1 > 0 && p.a_split == A_WHOLE) || p.dual_b) ptx::prefetch_tensormap(&tmB1);
    if (p.K1 > 0 || p.a_split != A_WHOLE) ptx::prefetch_tensormap(&tmA1);
    if (p.a_split != A_WHOLE) ptx::prefetch_tensormap(&tmA2);
    if (p.tma_out) ptx::prefetch_tensormap(&tmO0);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(tmem_slot, kTmemCols);
    ptx::tmem_relinquish_alloc_permit_pair();
  }
  ptx::tcgen05_fence_before_sync();
  __syncthreads();
  ptx::cluster_sync_all();  // the peer's barriers exist before anything signals them
  ptx::tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  grid_dependency_wait();  // barriers, tensor memory and descriptors were set up while the previous kernel drained

  constexpr int kBk = Geo<T>::kBk, kMnBox = Geo<T>::kMnBox, kBoxBytes = Geo<T>::kBoxBytes;
  const int nkb0 = (p.K0 + kBk - 1) / kBk;
  const int nkb1 = (p.K1 + kBk - 1) / kBk;
  const int nkb = nkb0 + nkb1 + (p.K2 + kBk - 1) / kBk;
  const int pair = blockIdx.x >> 1;
  const int npairs = gridDim.x >> 1;

  if (warp == 0 || warp == kPairProducerB) {
    // --------------------------------------------- TMA producers (A: warp 0, B: warp 10)
    // Two lanes in different warps share the issue work of a k-block: with MN-major operands a
    // k-block takes four tile loads per CTA, and one thread issuing all of them (plus the
    // barrier traffic) was within a factor ~1.4 of the 512 cycles the MMAs of a k-block take.
    if (lane == 0) {
      const bool do_a = warp == 0;
      const bool draws = p.sched != nullptr && do_a && leader;  // this thread hands out the tiles
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int next = -1;
      if (draws) {
        next = sched_draw(p);
        sched_publish(p, pair, 0, next);
      }
      for (int it = 0; ok; ++it) {
        int tile;
        if (draws) {
          tile = next;
          if (tile >= 0) {  // claim the following tile now: the others find it published early
            next = sched_draw(p);
            sched_publish(p, pair, it + 1, next);
          }
        } else {
          tile = sched_wait(p, pair, npairs, it, cta_abort, ST_PRODUCER);
        }
        if (tile < 0) break;
        int m_idx, n_idx;
        tile_coords(p, tile, &m_idx, &n_idx);
        const int m0 = m_idx * (2 * BM) + static_cast<int>(rank) * BM;
        const int n0 = p.dual_b ? n_idx * (BN / 2) : n_idx * BN + static_cast<int>(rank) * (BN / 2);
        for (int kb = 0; kb < nkb; ++kb) {
          if (!ptx::mbar_wait(&empty[stage], phase ^ 1u, cta_abort, p.status, ST_PRODUCER)) {
            ok = false;
            break;
          }
          const bool second = p.a_split == A_WHOLE && kb >= nkb0;
          uint8_t* sa = smem + stage * kStageBytes2;
          if (do_a) {
            if (leader) ptx::mbar_arrive_expect_tx(&full[stage], 2 * kStageBytes2);
            const ASource as = a_source(p, &tmA0, &tmA1, &tmA2, kb, nkb0, nkb1, m0, kBk);
            if (p.a_kmajor) {
              ptx::tma_load_2d_pair(sa, as.map, as.k, as.m, &full[stage]);
            } else {
#pragma unroll
              for (int j = 0; j < BM / kMnBox; ++j)
                ptx::tma_load_2d_pair(sa + j * kBoxBytes, as.map, as.m + j * kMnBox, as.k, &full[stage]);
            }
          } else {
            const int k0 = second ? (kb - nkb0) * kBk : kb * kBk;  // A_SPLIT_K: B's K range runs on
            const CUtensorMap* tb = p.dual_b ? (rank ? &tmB1 : &tmB0) : (second ? &tmB1 : &tmB0);
            uint8_t* sb = sa + kABytes;
            if (p.b_kmajor) {
              ptx::tma_load_2d_pair(sb, tb, k0, n0, &full[stage]);
            } else {
#pragma unroll
              for (int j = 0; j < (BN / 2) / kMnBox; ++j)
                ptx::tma_load_2d_pair(sb + j * kBoxBytes, tb, n0 + j * kMnBox, k0, &full[stage]);
            }
          }
          if (++stage == kStages2) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok || *cta_abort != 0) {
        const uint64_t t0 = ptx::globaltimer_ns();
        while (ptx::globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------- MMA issuer (leader only)
    if (lane == 0 && leader) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int it = 0; ok; ++it) {
        if (sched_wait(p, pair, npairs, it, cta_abort, ST_MMA_ACC) < 0) break;
        if (!ptx::mbar_wait(&tempty[acc], acc_phase ^ 1u, cta_abort, p.status, ST_MMA_ACC)) break;
        ptx::tcgen05_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < nkb; ++kb) {
          if (!ptx::mbar_wait(&full[stage], phase, cta_abort, p.status, ST_MMA_FULL)) {
            ok = false;
            break;
          }
          ptx::tcgen05_fence_after_sync();
          const uint32_t a_addr = ptx::smem_u32(smem + stage * kStageBytes2);
          const uint64_t a_desc = ptx::smem_desc(p.a_desc_hi, a_addr);
          const uint64_t b_desc = ptx::smem_desc(p.b_desc_hi, a_addr + kABytes);
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            if constexpr (sizeof(T) == 4)
              ptx::umma_tf32_pair(d_tmem, a_desc + static_cast<uint64_t>(kk * p.a_kstep),
                                  b_desc + static_cast<uint64_t>(kk * p.b_kstep), p.idesc,
                                  (kb | kk) != 0 ? 1u : 0u);
            else
              ptx::umma_f16_pair(d_tmem, a_desc + static_cast<uint64_t>(kk * p.a_kstep),
                                 b_desc + static_cast<uint64_t>(kk * p.b_kstep), p.idesc,
                                 (kb | kk) != 0 ? 1u : 0u);
          }
          ptx::umma_commit_pair(&empty[stage]);
          if (++stage == kStages2) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        ptx::umma_commit_pair(&tfull[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    int acc = 0;
    uint32_t acc_phase = 0;
    OutStage stg;
    stg.base = p.tma_out ? ptx::smem_u32(smem + kStages2 * kStageBytes2 + kCtrlBytes) +
                               static_cast<uint32_t>(warp - 2) * (2 * kStageOutBytes)
                         : 0u;
    stg.count = 0;
    for (int it = 0;; ++it) {
      int tile = 0;
      if (lane == 0) tile = sched_wait(p, pair, npairs, it, cta_abort, ST_EPILOGUE);
      tile = __shfl_sync(0xffffffffu, tile, 0);
      if (tile < 0) break;
      int m_idx, n_idx;
      tile_coords(p, tile, &m_idx, &n_idx);
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(&tfull[acc], acc_phase, cta_abort, p.status, ST_EPILOGUE)))
        break;
      ptx::tcgen05_fence_after_sync();
      const uint32_t taddr =
          tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BN);
      const int64_t row =
          static_cast<int64_t>(m_idx) * (2 * BM) + static_cast<int64_t>(rank) * BM + quarter * 32 + lane;
      if (EPI == EPI_PLAIN) epi_plain<T>(p, taddr, row, n_idx * BN, half, stg, &tmO0, &tmO1, &tmO2, lane);
      if (EPI == EPI_SWIGLU_FWD)
        epi_swiglu_fwd<T>(p, taddr, row, n_idx * (BN / 2), half, stg, &tmO0, &tmO1, &tmO2, lane);
      if (EPI == EPI_SWIGLU_BWD) epi_swiglu_bwd<T>(p, taddr, row, n_idx * BN, half, stg, &tmO0, &tmO1, lane);
      if (EPI == EPI_LCE) epi_lce<T>(p, taddr, row, n_idx * BN, n_idx, half, stg, &tmO0, lane);
      ptx::tcgen05_fence_before_sync();
      if (leader)
        ptx::mbar_arrive(&tempty[acc]);
      else
        ptx::mbar_arrive_cluster(&tempty[acc], 0);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (stg.base != 0 && lane == 0) ptx::bulk_wait_group<0>();
  }

  // ------------------------------------------------------------------ teardown
  ptx::tcgen05_fence_before_sync();
  __syncthreads();
  ptx::cluster_sync_all();  // both CTAs are done with tensor memory and with each other's barriers
  if (warp == 1) {
    ptx::tcgen05_fence_after_sync();
    ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

// ----------------------------------------------------------------------- host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// One operand as the caller describes it.
struct Operand {
  const void* ptr = nullptr;
  int kmajor = 1;    // 1: [mn, k] rows with k contiguous; 0: [k, mn] rows with mn contiguous
  int64_t mn = 0;    // extent along M (A) or N (B)
  int64_t k = 0;
  int64_t ld = 0;    // row stride in elements
  int box_mn = 0;    // rows of the K-major box (BM, BN or BN/2)
};

// A tensor map is a pure function of (address, extents, row stride, box, element type), so an
// encoded map can be reused for as long as the process lives, whatever has happened to the
// memory in between.  Each host thread keeps a small direct-mapped cache of the maps it has
// encoded (no locking; a training step asks for the same few hundred descriptions every time),
// which takes the driver's encode call - two to four per GEMM - off the launch path.
struct TmapKey {
  const void* ptr;
  int64_t mn, k, ld;
  int kmajor, box_mn, dtype;
  bool operator==(const TmapKey& o) const {
    return ptr == o.ptr && mn == o.mn && k == o.k && ld == o.ld && kmajor == o.kmajor &&
           box_mn == o.box_mn && dtype == o.dtype;
  }
};
constexpr int kTmapCacheSize = 1024;  // entries per thread (power of two)
struct TmapCache {
  TmapKey key[kTmapCacheSize];
  CUtensorMap map[kTmapCacheSize];
  bool used[kTmapCacheSize];
  uint64_t hits = 0, misses = 0;
  TmapCache() {
    for (int i = 0; i < kTmapCacheSize; ++i) used[i] = false;
  }
};
inline TmapCache& tmap_cache() {
  thread_local TmapCache* c = new TmapCache();  // lives as long as the thread's library use
  return *c;
}
inline size_t tmap_hash(const TmapKey& k) {
  uint64_t h = reinterpret_cast<uintptr_t>(k.ptr) * 0x9E3779B97F4A7C15ull;
  h ^= static_cast<uint64_t>(k.mn) * 0xC2B2AE3D27D4EB4Full + static_cast<uint64_t>(k.k) * 0x165667B19E3779F9ull;
  h ^= static_cast<uint64_t>(k.ld) * 0x27D4EB2F165667C5ull +
       static_cast<uint64_t>(k.kmajor * 4 + k.dtype + k.box_mn * 16);
  return static_cast<size_t>((h >> 29) & (kTmapCacheSize - 1));
}
inline bool& tmap_cache_enabled() {
  static bool on = true;
  return on;
}

int encode_tmap(CUtensorMap* tm, const Operand& o, int dtype, const char* what);

// `dtype`: BT_BF16 / BT_FP16 / BT_FP32 (fp32 operands feed the tensor cores as tf32).
inline int make_tmap(CUtensorMap* tm, const Operand& o, int dtype, const char* what) {
  if (!tmap_cache_enabled()) return encode_tmap(tm, o, dtype, what);
  const TmapKey key{o.ptr, o.mn, o.k, o.ld, o.kmajor, o.box_mn, dtype};
  TmapCache& c = tmap_cache();
  const size_t slot = tmap_hash(key);
  if (c.used[slot] && c.key[slot] == key) {
    ++c.hits;
    *tm = c.map[slot];
    return BT_OK;
  }
  ++c.misses;
  if (int rc = encode_tmap(tm, o, dtype, what)) return rc;
  c.key[slot] = key;
  c.map[slot] = *tm;
  c.used[slot] = true;
  return BT_OK;
}

inline int encode_tmap(CUtensorMap* tm, const Operand& o, int dtype, const char* what) {
  const int esize = dtype == BT_FP32 ? 4 : 2;
  const int row_elems = kRowBytes / esize;  // elements in one 128-byte row of a tile
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return BT_ERR_DRIVER;
  }
  if (!aligned16(o.ptr) || (o.ld * esize) % 16 != 0) {
    set_error("%s: operand must be 16-byte aligned with a row stride that is a multiple of %d elements",
              what, 16 / esize);
    return BT_ERR_ARG;
  }
  cuuint64_t dims[2];
  cuuint32_t box[2];
  if (o.kmajor == 2) {  // a result tensor [rows = mn, cols = k]: 32 x 32 boxes of 16-bit elements
    dims[0] = static_cast<cuuint64_t>(o.k);
    dims[1] = static_cast<cuuint64_t>(o.mn);
    box[0] = 32;
    box[1] = 32;
  } else if (o.kmajor) {
    dims[0] = static_cast<cuuint64_t>(o.k);
    dims[1] = static_cast<cuuint64_t>(o.mn);
    box[0] = static_cast<cuuint32_t>(row_elems);
    box[1] = static_cast<cuuint32_t>(o.box_mn);
  } else {
    dims[0] = static_cast<cuuint64_t>(o.mn);
    dims[1] = static_cast<cuuint64_t>(o.k);
    box[0] = static_cast<cuuint32_t>(row_elems);
    box[1] = static_cast<cuuint32_t>(row_elems);  // k-block = 128 bytes of K as well
  }
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(o.ld) * esize};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = dtype == BT_BF16   ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                 : dtype == BT_FP16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                    : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  const CUresult r = fn(tm, dt, 2, const_cast<void*>(o.ptr), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE,
                        o.kmajor == 2 ? CU_TENSOR_MAP_SWIZZLE_64B
                        : (dtype == BT_FP32 && !o.kmajor) ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                                                          : CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("%s: cuTensorMapEncodeTiled failed with CUresult %d (dims %llu x %llu, ld %lld)", what,
              static_cast<int>(r), (unsigned long long)dims[0], (unsigned long long)dims[1],
              (long long)o.ld);
    return BT_ERR_DRIVER;
  }
  return BT_OK;
}

template <int EPI, typename T>
int launch_t(const CUtensorMap& a0, const CUtensorMap& b0, const CUtensorMap& a1,
             const CUtensorMap& b1, const CUtensorMap& a2, const CUtensorMap (&o)[3], const Params& p,
             cudaStream_t s) {
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  auto* kern = gemm_kernel<EPI, T>;
  std::call_once(once, [&] {
    attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  });
  if (attr_err != cudaSuccess) {
    set_error("gemm: cannot reserve %d bytes of shared memory: %s", kSmemBytes,
              cudaGetErrorString(attr_err));
    return BT_ERR_LAUNCH;
  }
  const int grid = p.num_tiles < sm_count() ? p.num_tiles : sm_count();
  BT_CHECK_LAUNCHED(launch_dependent(kern, dim3(grid), dim3(kThreads), kSmemBytes, s, a0, b0, a1, b1, a2, o[0],
                                     o[1], o[2], p),
                    "gemm_kernel");
  return BT_OK;
}

// 1 (default): 16-bit results are staged in shared memory and written with tile stores;
// 0: every epilogue thread stores its own row pieces.
inline int& tma_out_mode() {
  static int mode = 1;
  return mode;
}

// Row tiles walked per column tile before the walk moves on (tile rasterisation); 0 = the
// built-in choice.
inline int& group_m_override() {
  static int g = 0;
  return g;
}

// 0 (default): tiles are dealt round-robin; 1: CTA pairs draw them from a global counter.
inline int& dynamic_tiles() {
  static int mode = 0;
  return mode;
}

// Device address of the scheduler pool on the current device (looked up once per device).
inline unsigned long long* sched_pool() {
  static std::mutex mu;
  static unsigned long long* pools[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (pools[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_tile_sched) != cudaSuccess) return nullptr;
    pools[dev] = static_cast<unsigned long long*>(ptr);
  }
  return pools[dev];
}

// Slot of the scheduler pool owned by (current device, stream): handed out first come, first
// served, kept for the life of the process; -1 when all kSchedSlots are taken on this device.
inline int sched_slot_of(cudaStream_t s) {
  static std::mutex mu;
  static cudaStream_t owner[64][kSchedSlots];
  static int used[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < used[dev]; ++i)
    if (owner[dev][i] == s) return i;
  if (used[dev] >= kSchedSlots) return -1;
  owner[dev][used[dev]] = s;
  return used[dev]++;
}

template <int EPI, typename T>
int launch_pair_t(const CUtensorMap& a0, const CUtensorMap& b0, const CUtensorMap& a1,
                  const CUtensorMap& b1, const CUtensorMap& a2, const CUtensorMap (&o)[3],
                  const Params& p, cudaStream_t s) {
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  auto* kern = gemm_kernel_pair<EPI, T>;
  std::call_once(once, [&] {
    attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes2);
  });
  if (attr_err != cudaSuccess) {
    set_error("gemm: cannot reserve %d bytes of shared memory: %s", kSmemBytes2,
              cudaGetErrorString(attr_err));
    return BT_ERR_LAUNCH;
  }
  const int max_pairs = sm_count() / 2;
  const int pairs = p.num_tiles < max_pairs ? p.num_tiles : max_pairs;
  Params q = p;
  q.sched = nullptr;
  if (dynamic_tiles() != 0 && pairs <= kSchedMaxPairs && p.num_tiles > pairs) {
    // This stream's slot of the scheduler pool, cleared on the stream ahead of the kernel.  A
    // slot belongs to one (device, stream): within a stream the memset is ordered after the
    // previous launch, so it can never clear a ring that a kernel is still reading, and launches
    // on other streams use other slots.  A stream that finds no free slot deals its tiles
    // round-robin (q.sched stays null).
    const int slot = sched_slot_of(s);
    if (slot >= 0) {
      unsigned long long* pool = sched_pool();
      if (pool == nullptr) {
        set_error("gemm: cannot locate the tile-scheduler pool");
        return BT_ERR_DRIVER;
      }
      q.sched = pool + static_cast<size_t>(slot) * kSchedWords;
      const cudaError_t me =
          cudaMemsetAsync(q.sched, 0, sizeof(unsigned long long) * (1 + pairs * kSchedRing), s);
      if (me != cudaSuccess) {
        set_error("gemm: clearing the tile scheduler failed: %s", cudaGetErrorString(me));
        return BT_ERR_LAUNCH;
      }
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs), 1, 1);
  cfg.blockDim = dim3(kThreadsPair, 1, 1);
  cfg.dynamicSmemBytes = kSmemBytes2;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = dependent_launch_mode() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a0, b0, a1, b1, a2, o[0], o[1], o[2], q);
  if (e != cudaSuccess) {
    set_error("gemm_kernel_pair: %s", cudaGetErrorString(e));
    return BT_ERR_LAUNCH;
  }
  return BT_OK;
}

// 0: one CTA per 128 x 256 tile (cta_group::1); 1: CTA pairs on 256 x 256 tiles (cta_group::2).
inline int& pair_mode() {
  static int mode = 1;
  return mode;
}

// Describes one GEMM launch; pair 1 and b1 are optional.
struct Launch {
  Operand a0, b0, a1, b1, a2;
  bool dual_b = false;    // b1 is the second half of the B tile (same K range as pair 0)
  bool two_pairs = false; // (a1, b1) is a second contraction into the same accumulator
  int a_split = A_WHOLE;  // A_SPLIT_K / A_SPLIT_M: A is (a0, a1, a2), B is b0 alone
  int dtype = BT_BF16;    // storage of the operands: BT_BF16, BT_FP16 or BT_FP32 (tf32 math)
  Params p{};
};

// cuTensorMapEncodeTiled is a driver call and wants a current context on the calling
// thread; a thread that has made no runtime call yet (an autograd worker, say) has
// none bound, so bind the primary context of the current device once per thread.
inline void bind_context_once() {
  thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
}

template <int EPI>
int launch(Launch& L, cudaStream_t s) {
  bind_context_once();
  Params& p = L.p;
  const bool pair = pair_mode() != 0;
  const int n_tile = L.dual_b ? BN / 2 : BN;
  p.K0 = static_cast<int>(L.a0.k);
  p.K1 = L.two_pairs ? static_cast<int>(L.a1.k) : 0;
  p.K2 = 0;
  p.a_split = L.a_split;
  p.m_seg0 = p.m_seg1 = 0;
  if (L.a_split != A_WHOLE) {
    const int kbk = kRowBytes / (L.dtype == BT_FP32 ? 4 : 2);
    const int tile_m = pair ? 2 * BM : BM;
    if (L.two_pairs || L.dual_b || L.a1.kmajor != L.a0.kmajor || L.a2.kmajor != L.a0.kmajor) {
      set_error("gemm: a split A operand excludes the other main-loop modes and needs one layout");
      return BT_ERR_ARG;
    }
    if (L.a_split == A_SPLIT_K) {
      if (L.a0.k % kbk != 0 || L.a1.k % kbk != 0 || L.a1.k <= 0 || L.a2.k <= 0 ||
          L.b0.k != L.a0.k + L.a1.k + L.a2.k) {
        set_error("gemm: K-split A needs K and K1 in whole k-blocks of %d and B spanning K + K1 + K2", kbk);
        return BT_ERR_ARG;
      }
      p.K1 = static_cast<int>(L.a1.k);
      p.K2 = static_cast<int>(L.a2.k);
    } else {
      if (L.a0.mn % tile_m != 0 || L.a1.mn % tile_m != 0 || L.a1.mn <= 0 || L.a2.mn <= 0 ||
          L.a0.mn + L.a1.mn + L.a2.mn != p.M || L.a1.k != L.a0.k || L.a2.k != L.a0.k) {
        set_error("gemm: M-split A needs segments in whole tiles of %d rows that add up to M", tile_m);
        return BT_ERR_ARG;
      }
      p.m_seg0 = static_cast<int>(L.a0.mn);
      p.m_seg1 = static_cast<int>(L.a1.mn);
    }
  }
  p.tiles_m = static_cast<int>(ceil_div(p.M, pair ? 2 * BM : BM));
  p.tiles_n = static_cast<int>(ceil_div(p.N, n_tile));
  const int64_t nt = static_cast<int64_t>(p.tiles_m) * p.tiles_n;
  if (nt <= 0 || nt > 0x7fffffff || p.K0 <= 0) {
    set_error("gemm: empty or oversized problem (M=%d N=%d K=%d)", p.M, p.N, p.K0);
    return BT_ERR_ARG;
  }
  p.num_tiles = static_cast<int>(nt);
  // Rasterisation: CTAs that run at the same time share operand tiles through L2.  With a short
  // contraction the A panel of 16 row tiles (16 x 256 rows x K) stays in L2 while the walk
  // crosses all column tiles, so B is fetched once per 16 row tiles.  With a long contraction
  // that panel does not fit (K x element size > 16 KB <=> more than 64 MB) and nothing is
  // reused between waves; then a wave of 74 tiles should be as square as possible (8 x 9
  // tiles touch 17 panels, 16 x 4.6 touch 21).  Measured on the fused loss (dx has K = 151936):
  // 49.9 ms with 8 against 51-52.5 ms with 16; the MLP block (K <= 24576) is indifferent.
  const int64_t k_total = L.a_split == A_SPLIT_K ? L.b0.k : (L.a0.k + (L.two_pairs ? L.a1.k : 0));
  const int esz = L.dtype == BT_FP32 ? 4 : 2;
  p.group_m = group_m_override() > 0 ? group_m_override() : (k_total * esz > 16384 ? kGroupM / 2 : kGroupM);
  p.a_kmajor = L.a0.kmajor;
  p.b_kmajor = L.b0.kmajor;
  p.dual_b = L.dual_b ? 1 : 0;
  const int esize = L.dtype == BT_FP32 ? 4 : 2;
  const int box_bytes = (kRowBytes / esize) * kRowBytes;  // one MN-major box: 128-byte rows, 128 bytes of K
  const uint32_t fmt = L.dtype == BT_FP16 ? 0u : (L.dtype == BT_BF16 ? 1u : 2u);
  p.idesc = ptx::make_idesc(fmt, !L.a0.kmajor, !L.b0.kmajor, pair ? 2 * BM : BM, BN);
  p.a_desc_hi = ptx::make_smem_desc_hi(L.a0.kmajor != 0, static_cast<uint32_t>(box_bytes),
                                       esize == 4 && !L.a0.kmajor);
  p.b_desc_hi = ptx::make_smem_desc_hi(L.b0.kmajor != 0, static_cast<uint32_t>(box_bytes),
                                       esize == 4 && !L.b0.kmajor);
  // one MMA consumes 32 bytes of K: 32 bytes along a K-major row, or 32/esize rows of 128 bytes
  const uint32_t mn_step = static_cast<uint32_t>((32 / esize) * kRowBytes) >> 4;
  p.a_kstep = L.a0.kmajor ? (32u >> 4) : mn_step;
  p.b_kstep = L.b0.kmajor ? (32u >> 4) : mn_step;
  // K-major boxes: a CTA of a pair stages 128 rows of A and 128 of the tile's 256 B rows
  const int b_box = pair ? BN / 2 : n_tile;
  L.a0.box_mn = BM;
  L.b0.box_mn = b_box;
  CUtensorMap ta0, tb0, ta1, tb1, ta2;
  int rc;
  if ((rc = make_tmap(&ta0, L.a0, L.dtype, "gemm A")) != BT_OK) return rc;
  if ((rc = make_tmap(&tb0, L.b0, L.dtype, "gemm B")) != BT_OK) return rc;
  ta1 = ta0;
  tb1 = tb0;
  ta2 = ta0;
  if (L.a_split != A_WHOLE) {
    L.a1.box_mn = BM;
    L.a2.box_mn = BM;
    if ((rc = make_tmap(&ta1, L.a1, L.dtype, "gemm A1")) != BT_OK) return rc;
    if ((rc = make_tmap(&ta2, L.a2, L.dtype, "gemm A2")) != BT_OK) return rc;
  } else if (L.two_pairs) {
    if (L.a1.kmajor != L.a0.kmajor || L.b1.kmajor != L.b0.kmajor) {
      set_error("gemm: both operand pairs must share their layouts");
      return BT_ERR_ARG;
    }
    L.a1.box_mn = BM;
    L.b1.box_mn = b_box;
    if ((rc = make_tmap(&ta1, L.a1, L.dtype, "gemm A1")) != BT_OK) return rc;
    if ((rc = make_tmap(&tb1, L.b1, L.dtype, "gemm B1")) != BT_OK) return rc;
  } else if (L.dual_b) {
    if (!L.b0.kmajor || !L.b1.kmajor) {
      set_error("gemm: dual-B mode needs K-major B operands");
      return BT_ERR_ARG;
    }
    L.b1.box_mn = b_box;
    if ((rc = make_tmap(&tb1, L.b1, L.dtype, "gemm B1")) != BT_OK) return rc;
  }
  // 16-bit results with 16-byte aligned rows leave through shared memory and tile stores
  CUtensorMap to[3];
  to[0] = to[1] = to[2] = ta0;  // placeholders when unused
  p.tma_out = 0;
  if (tma_out_mode() != 0 && L.dtype != BT_FP32 && !p.out_fp32 && p.vec_ok) {
    struct Out {
      void* ptr;
      int64_t rows, cols, ld;
    } outs[3] = {};
    int n_out = 0;
    if (EPI == EPI_PLAIN) {
      if (p.n_seg0 > 0) {
        outs[0] = {p.out, p.M, p.n_seg0, p.ldo};
        outs[1] = {p.out1, p.M, p.n_seg1, p.ldo1};
        outs[2] = {p.out2, p.M, p.N - p.n_seg0 - p.n_seg1, p.ldo2};
        n_out = 3;
      } else {
        outs[0] = {p.out, p.M, p.N, p.ldo};
        n_out = 1;
      }
    } else if (EPI == EPI_SWIGLU_FWD) {
      outs[0] = {p.gate, p.M, p.N, p.ld_act};
      outs[1] = {p.up, p.M, p.N, p.ld_act};
      outs[2] = {p.h, p.M, p.N, p.ld_act};
      n_out = 3;
    } else if (EPI == EPI_SWIGLU_BWD) {
      outs[0] = {p.out, p.M, p.N, p.ldo};
      outs[1] = {p.h, p.M, p.N, p.ldo};
      n_out = 2;
    } else {
      outs[0] = {p.out, p.M, p.N, p.ldo};
      n_out = 1;
    }
    bool ok = true;
    for (int i = 0; i < n_out && ok; ++i) {
      Operand o;
      o.ptr = outs[i].ptr;
      o.kmajor = 2;  // marks a result map (box 32 x 32, 64-byte swizzle) in the cache key
      o.mn = outs[i].rows;
      o.k = outs[i].cols;
      o.ld = outs[i].ld;
      o.box_mn = 32;
      ok = outs[i].ptr != nullptr && make_tmap(&to[i], o, L.dtype, "gemm result") == BT_OK;
    }
    p.tma_out = ok ? 1 : 0;
  }
  if (pair) {
    switch (L.dtype) {
      case BT_BF16: return launch_pair_t<EPI, __nv_bfloat16>(ta0, tb0, ta1, tb1, ta2, to, p, s);
      case BT_FP16: return launch_pair_t<EPI, __half>(ta0, tb0, ta1, tb1, ta2, to, p, s);
      default: return launch_pair_t<EPI, float>(ta0, tb0, ta1, tb1, ta2, to, p, s);
    }
  }
  switch (L.dtype) {
    case BT_BF16: return launch_t<EPI, __nv_bfloat16>(ta0, tb0, ta1, tb1, ta2, to, p, s);
    case BT_FP16: return launch_t<EPI, __half>(ta0, tb0, ta1, tb1, ta2, to, p, s);
    default: return launch_t<EPI, float>(ta0, tb0, ta1, tb1, ta2, to, p, s);
  }
}

}  // namespace gemm
}  // namespace bt

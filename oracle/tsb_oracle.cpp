// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// CPU oracle: a plain C++ restatement of what triton-shared's reference CPU
// backend computes when it executes a lowered kernel.  Only tests, the smoke
// check and the benchmark's CPU-baseline legs may load this library; the GPU
// product path never does.
//
// The reference itself cannot be built in this environment (it needs
// triton-shared-opt, mlir-opt, mlir-translate and llc; backend/compiler.py:16-27,
// 58, 81-122, 172-173), so this file restates the lowered loops from the sources
// cited at each function (paths inside microsoft/triton-shared).  Pins:
//   * block copy: checked against the reference's own memrefCopy compiled from
//     backend/include/ExecutionEngine/CRunnerUtils.cpp (oracle/_ref, see Makefile);
//   * load/store/mask semantics: checked against the exact known answers in
//     python/examples/test_mask.py:39,58,64, test_load_2d_tensor_block.py:76-78,
//     test_swap.py:34-44, test_splat.py:24-41;
//   * kernel arithmetic: checked against Triton's own CPU interpreter running
//     the reference's example kernels (fixtures under tests/golden).
// The reference's tests hold no numeric golden vectors for vec-add or layernorm
// (test_vec_add.py:63-69 and test_layernorm.py:129-136 only print), so for
// those two the parity pin is the interpreter fixture, not a reference output.
//
// Build: g++ -O2 -ffp-contract=off (no contraction: the reference lowers mul and
// add as separate ops and llc is run without fast-math, backend/compiler.py:172).
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <vector>

#include <functional>
#include <thread>

namespace {

// --- 16-bit float helpers ---------------------------------------------------
inline float f16_to_f32(uint16_t h) {
  _Float16 v;
  memcpy(&v, &h, 2);
  return (float)v;  // arith.extf: exact
}
inline uint16_t f32_to_f16(float f) {
  _Float16 v = (_Float16)f;  // arith.truncf: round to nearest even
  uint16_t h;
  memcpy(&h, &v, 2);
  return h;
}
inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);  // quiet NaN
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;  // round to nearest even
  return (uint16_t)(u >> 16);
}
enum { ORC_F32 = 0, ORC_F16 = 1, ORC_BF16 = 2 };
inline float ld16(const uint16_t *p, int dt) { return dt == ORC_F16 ? f16_to_f32(*p) : bf16_to_f32(*p); }
inline uint16_t st16(float v, int dt) { return dt == ORC_F16 ? f32_to_f16(v) : f32_to_bf16(v); }

// Access size of one masked dim.
// lib/Analysis/MaskAnalysis.cpp:583-585: dims = max(min(end, bound), start) - start,
// all signed 64-bit (OpFoldResultUtils.cpp:320,348).
inline int64_t mask_dim(int64_t start, int64_t size, int64_t bound) {
  int64_t end = start + size;
  int64_t m = std::min(end, bound);
  m = std::max(m, start);
  return m - start;
}

// Element-by-element strided copy with an index odometer, innermost dim fastest:
// backend/include/ExecutionEngine/CRunnerUtils.cpp:58-113.
void strided_copy(int64_t esize, int rank, const int64_t *sizes, const char *src,
                  const int64_t *sstr, char *dst, const int64_t *dstr) {
  for (int d = 0; d < rank; ++d)
    if (sizes[d] == 0) return;
  if (rank == 0) {
    memcpy(dst, src, (size_t)esize);
    return;
  }
  std::vector<int64_t> idx((size_t)rank, 0);
  int64_t r = 0, w = 0;
  for (;;) {
    memcpy(dst + w * esize, src + r * esize, (size_t)esize);
    int d = rank - 1;
    for (; d >= 0; --d) {
      ++idx[d];
      r += sstr[d];
      w += dstr[d];
      if (idx[d] != sizes[d]) break;
      if (d == 0) return;
      idx[d] = 0;
      r -= sizes[d] * sstr[d];
      w -= sizes[d] * dstr[d];
    }
  }
}

void dense_strides(int rank, const int64_t *sizes, int64_t *out) {
  int64_t s = 1;
  for (int d = rank - 1; d >= 0; --d) {
    out[d] = s;
    s *= sizes[d];
  }
}

}  // namespace

extern "C" {

int64_t orc_mask_dim(int64_t start, int64_t size, int64_t bound) { return mask_dim(start, size, bound); }

// Strided copy exposed for the comparison with the reference's memrefCopy.
void orc_strided_copy(int64_t esize, int rank, const int64_t *sizes, const void *src,
                      const int64_t *src_strides, void *dst, const int64_t *dst_strides) {
  strided_copy(esize, rank, sizes, (const char *)src, src_strides, (char *)dst, dst_strides);
}

// Structured block load into a dense row-major buffer `dst` of the full block.
//   view = reinterpret_cast(base, offset, sizes, strides)     StructuredToMemref.cpp:528-551
//   unmasked: copy the whole view                              :748-792
//   masked  : if `other` and some dims[d] < sizes[d], fill the whole buffer with
//             other (:192-224, :809-813); then copy subview[0..][dims][1..] (:841-845).
// `dims` == NULL means unmasked.  Lanes the reference leaves uninitialised (masked,
// no `other`) are zeroed here so that results are reproducible.
void orc_block_load(const void *base, int64_t esize, int rank, const int64_t *sizes,
                    const int64_t *strides, int64_t offset, const int64_t *dims, const void *other,
                    void *dst) {
  int64_t total = 1;
  for (int d = 0; d < rank; ++d) total *= sizes[d];
  std::vector<int64_t> dstr((size_t)std::max(rank, 1));
  dense_strides(rank, sizes, dstr.data());
  const char *src = (const char *)base + offset * esize;
  if (!dims) {
    strided_copy(esize, rank, sizes, src, strides, (char *)dst, dstr.data());
    return;
  }
  bool shorter = false;
  for (int d = 0; d < rank; ++d) shorter = shorter || dims[d] < sizes[d];
  if (other && shorter) {
    for (int64_t i = 0; i < total; ++i) memcpy((char *)dst + i * esize, other, (size_t)esize);
  } else if (!other) {
    memset(dst, 0, (size_t)(total * esize));
  }
  strided_copy(esize, rank, dims, src, strides, (char *)dst, dstr.data());
}

// Structured block store from a dense row-major buffer: writes value[0:dims] to
// view[0:dims] (extract_slice + subview + materialize_in_destination,
// StructuredToMemref.cpp:1163-1196). dims == NULL: whole block.
void orc_block_store(void *base, int64_t esize, int rank, const int64_t *sizes,
                     const int64_t *strides, int64_t offset, const int64_t *dims, const void *src) {
  std::vector<int64_t> sstr((size_t)std::max(rank, 1));
  dense_strides(rank, sizes, sstr.data());
  char *dst = (char *)base + offset * esize;
  strided_copy(esize, rank, dims ? dims : sizes, (const char *)src, sstr.data(), dst, strides);
}

// Program loop of the reference launcher (backend/driver.py:116-133): serial
// with threads == 1.  With threads > 1 the programs are split into contiguous
// chunks, one per host thread, which mirrors the launcher's own parallel mode
// (`#pragma omp parallel for`, driver.py:119-121); programs are independent, so
// results do not depend on the thread count.
static void program_loop(int64_t lo, int64_t hi, int threads, const std::function<void(int64_t)> &body) {
  if (threads <= 1 || hi - lo <= 1) {
    for (int64_t p = lo; p < hi; ++p) body(p);
    return;
  }
  const int64_t n = hi - lo;
  const int64_t t = std::min<int64_t>(threads, n);
  std::vector<std::thread> pool;
  for (int64_t k = 0; k < t; ++k) {
    const int64_t a = lo + n * k / t, b = lo + n * (k + 1) / t;
    pool.emplace_back([a, b, &body]() {
      for (int64_t p = a; p < b; ++p) body(p);
    });
  }
  for (auto &th : pool) th.join();
}
#define ORC_PROGRAM_LOOP(pid, lo, hi, threads) program_loop(lo, hi, threads, [&](int64_t pid)
#define ORC_END_LOOP )

// ---------------------------------------------------------------------------
// config 1: masked vector add (python/examples/test_vec_add.py:8-34; lowered
// form test/Conversion/StructuredToMemref/kernel-01-vector-add.mlir:29-61).
void orc_vec_add(const float *x, const float *y, float *z, int64_t n, int64_t block,
                 int64_t pid_lo, int64_t pid_hi, int threads) {
  if (threads < 1) threads = 1;
  ORC_PROGRAM_LOOP(pid, pid_lo, pid_hi, threads) {
    std::vector<float> bx((size_t)block), by((size_t)block), bz((size_t)block);
    const int64_t start = pid * block;
    const int64_t dim = mask_dim(start, block, n);
    const int64_t one = 1;
    orc_block_load(x, 4, 1, &block, &one, start, &dim, nullptr, bx.data());
    orc_block_load(y, 4, 1, &block, &one, start, &dim, nullptr, by.data());
    for (int64_t l = 0; l < block; ++l) bz[(size_t)l] = bx[(size_t)l] + by[(size_t)l];  // linalg.generic addf, all lanes
    orc_block_store(z, 4, 1, &block, &one, start, &dim, bz.data());
  } ORC_END_LOOP;
}

// ---------------------------------------------------------------------------
// config 2: fused row softmax (python/examples/test_softmax.py:8-29; lowered form
// test/Conversion/StructuredToMemref/kernel-02-fused-softmax.mlir:50-90).
// Reductions are left-to-right folds acc = op(x_i, acc) from the identity
// (ConversionPatterns.hpp:1227-1278, 1395-1407).
void orc_softmax(float *out, const float *in, int64_t in_stride, int64_t out_stride,
                 int64_t n_cols, int64_t block, int64_t row_lo, int64_t row_hi, int threads) {
  if (threads < 1) threads = 1;
  ORC_PROGRAM_LOOP(row, row_lo, row_hi, threads) {
    std::vector<float> b((size_t)block), e((size_t)block), o((size_t)block);
    const int64_t dim = mask_dim(0, block, n_cols);
    const int64_t one = 1;
    const float ninf = -INFINITY;
    orc_block_load(in, 4, 1, &block, &one, row * in_stride, &dim, &ninf, b.data());
    float m = -INFINITY;
    for (int64_t l = 0; l < block; ++l) m = fmaxf(b[(size_t)l], m);  // arith.maxnumf
    for (int64_t l = 0; l < block; ++l) e[(size_t)l] = b[(size_t)l] - m;
    for (int64_t l = 0; l < block; ++l) e[(size_t)l] = expf(e[(size_t)l]);  // math.exp -> libm
    float s = 0.f;
    for (int64_t l = 0; l < block; ++l) s = e[(size_t)l] + s;
    for (int64_t l = 0; l < block; ++l) o[(size_t)l] = e[(size_t)l] / s;
    orc_block_store(out, 4, 1, &block, &one, row * out_stride, &dim, o.data());
  } ORC_END_LOOP;
}

// ---------------------------------------------------------------------------
// config 3: LayerNorm forward (python/examples/test_layernorm.py:29-76; lowered
// form test/Conversion/StructuredToMemref/kernel-05-layer-norm-fwd.mlir).
// io_dtype: ORC_F16 / ORC_BF16 / ORC_F32 for X, Y, W, B.
void orc_layernorm_fwd(const void *X, void *Y, const void *W, const void *B, float *Mean,
                       float *Rstd, int64_t stride, int64_t N, float eps, int64_t block,
                       int io_dtype, int64_t row_lo, int64_t row_hi, int threads) {
  if (threads < 1) threads = 1;
  const int64_t es = io_dtype == ORC_F32 ? 4 : 2;
  auto widen = [&](const void *buf, int64_t l) -> float {
    return io_dtype == ORC_F32 ? ((const float *)buf)[l] : ld16((const uint16_t *)buf + l, io_dtype);
  };
  ORC_PROGRAM_LOOP(row, row_lo, row_hi, threads) {
    std::vector<char> bx((size_t)(block * es)), bw((size_t)(block * es)), bb((size_t)(block * es)),
        by((size_t)(block * es));
    std::vector<float> acc((size_t)block, 0.f);
    const int64_t one = 1;
    const char zero[4] = {0, 0, 0, 0};
    // loop 1: lane accumulators of x (masked lanes read other = 0)
    for (int64_t off = 0; off < N; off += block) {
      const int64_t dim = mask_dim(off, block, N);
      orc_block_load(X, es, 1, &block, &one, row * stride + off, &dim, zero, bx.data());
      for (int64_t l = 0; l < block; ++l) acc[(size_t)l] = acc[(size_t)l] + widen(bx.data(), l);
    }
    float s = 0.f;
    for (int64_t l = 0; l < block; ++l) s = acc[(size_t)l] + s;
    const float mean = s / (float)(int32_t)N;  // arith.sitofp + arith.divf
    // loop 2: lane accumulators of (x-mean)^2 with masked lanes forced to 0
    std::fill(acc.begin(), acc.end(), 0.f);
    for (int64_t off = 0; off < N; off += block) {
      const int64_t dim = mask_dim(off, block, N);
      orc_block_load(X, es, 1, &block, &one, row * stride + off, &dim, zero, bx.data());
      for (int64_t l = 0; l < block; ++l) {
        float d = widen(bx.data(), l) - mean;
        d = (off + l < N) ? d : 0.f;  // arith.select on the mask
        acc[(size_t)l] = acc[(size_t)l] + d * d;
      }
    }
    float q = 0.f;
    for (int64_t l = 0; l < block; ++l) q = acc[(size_t)l] + q;
    const float var = q / (float)(int32_t)N;
    const float rstd = 1.0f / sqrtf(var + eps);
    if (Mean) Mean[row] = mean;  // scalar tt.store (UnstructuredToMemrefPass.cpp:71-158)
    if (Rstd) Rstd[row] = rstd;
    // loop 3: normalise, scale, shift; one rounding per op, no contraction
    for (int64_t off = 0; off < N; off += block) {
      const int64_t dim = mask_dim(off, block, N);
      orc_block_load(W, es, 1, &block, &one, off, &dim, nullptr, bw.data());
      orc_block_load(B, es, 1, &block, &one, off, &dim, nullptr, bb.data());
      orc_block_load(X, es, 1, &block, &one, row * stride + off, &dim, zero, bx.data());
      for (int64_t l = 0; l < block; ++l) {
        float xh = (widen(bx.data(), l) - mean) * rstd;
        float y = xh * widen(bw.data(), l);
        y = y + widen(bb.data(), l);
        if (io_dtype == ORC_F32) ((float *)by.data())[l] = y;
        else ((uint16_t *)by.data())[l] = st16(y, io_dtype);
      }
      orc_block_store(Y, es, 1, &block, &one, row * stride + off, &dim, by.data());
    }
  } ORC_END_LOOP;
}

// ---------------------------------------------------------------------------
// config 4: blocked matmul via tt.dot (python/examples/test_matmul.py:34-108;
// lowered loop test/Conversion/StructuredToMemref/kernel-03-matrix-multiplication.mlir:157-204).
// Per K-step: P = A_blk * B_blk from zero with k ascending (linalg.matmul), then
// acc = acc + P (MatmulConverter, ConversionPatterns.hpp:1159-1199); one rounding
// to the output type at the end.  A/B block loads are masked to the valid M/N/K
// extents with other = 0.  tile_of_pid holds (tile_m, tile_n) per program.
void orc_matmul(const uint16_t *A, const uint16_t *Bm, uint16_t *C, int dtype, int64_t M, int64_t N,
                int64_t K, int64_t sam, int64_t sak, int64_t sbk, int64_t sbn, int64_t scm,
                int64_t scn, int64_t BM, int64_t BN, int64_t BK, const int32_t *tile_of_pid,
                int64_t pid_lo, int64_t pid_hi, int threads) {
  if (threads < 1) threads = 1;
  ORC_PROGRAM_LOOP(pid, pid_lo, pid_hi, threads) {
    const int64_t tm = tile_of_pid[2 * pid], tn = tile_of_pid[2 * pid + 1];
    std::vector<uint16_t> a((size_t)(BM * BK)), b((size_t)(BK * BN)), c((size_t)(BM * BN));
    std::vector<float> af((size_t)(BM * BK)), bf((size_t)(BK * BN)), acc((size_t)(BM * BN), 0.f),
        P((size_t)(BM * BN));
    const uint16_t zero = 0;
    for (int64_t k0 = 0; k0 < K; k0 += BK) {
      const int64_t asz[2] = {BM, BK}, astr[2] = {sam, sak};
      const int64_t adim[2] = {mask_dim(tm * BM, BM, M), mask_dim(k0, BK, K)};
      orc_block_load(A, 2, 2, asz, astr, tm * BM * sam + k0 * sak, adim, &zero, a.data());
      const int64_t bsz[2] = {BK, BN}, bstr[2] = {sbk, sbn};
      const int64_t bdim[2] = {mask_dim(k0, BK, K), mask_dim(tn * BN, BN, N)};
      orc_block_load(Bm, 2, 2, bsz, bstr, k0 * sbk + tn * BN * sbn, bdim, &zero, b.data());
      for (size_t i = 0; i < a.size(); ++i) af[i] = ld16(&a[i], dtype);
      for (size_t i = 0; i < b.size(); ++i) bf[i] = ld16(&b[i], dtype);
      std::fill(P.begin(), P.end(), 0.f);
      // i-k-j order gives the same per-element sum order as the i-j-k nest
      // (k ascending for every (i,j)) and is far faster on a CPU.
      for (int64_t i = 0; i < BM; ++i)
        for (int64_t k = 0; k < BK; ++k) {
          const float av = af[(size_t)(i * BK + k)];
          const float *brow = &bf[(size_t)(k * BN)];
          float *prow = &P[(size_t)(i * BN)];
          for (int64_t j = 0; j < BN; ++j) prow[j] = prow[j] + av * brow[j];
        }
      for (size_t i = 0; i < acc.size(); ++i) acc[i] = acc[i] + P[i];
    }
    for (size_t i = 0; i < acc.size(); ++i) c[i] = st16(acc[i], dtype);
    const int64_t csz[2] = {BM, BN}, cstr[2] = {scm, scn};
    const int64_t cdim[2] = {mask_dim(tm * BM, BM, M), mask_dim(tn * BN, BN, N)};
    orc_block_store(C, 2, 2, csz, cstr, tm * BM * scm + tn * BN * scn, cdim, c.data());
  } ORC_END_LOOP;
}

// ---------------------------------------------------------------------------
// config 5: strided masked 2-D reduction.  One program per block of BM rows; a
// loop over column blocks of BN loads the ragged block with strides
// [stride_m, stride_n] and other = 0 (masked_ldst_2d.mlir:76-99), sums it along
// axis 1 (reducesum_512_256_f32_axis1.mlir: transpose, then a fold over the
// reduced axis with j ascending) and adds the block's row sums to the running
// row sums; a masked 1-D store writes them.
void orc_reduce_rows(const float *x, float *out, int64_t M, int64_t n_valid, int64_t stride_m,
                     int64_t stride_n, int64_t BM, int64_t BN, int64_t pid_lo, int64_t pid_hi,
                     int threads) {
  if (threads < 1) threads = 1;
  ORC_PROGRAM_LOOP(pid, pid_lo, pid_hi, threads) {
    std::vector<float> blk((size_t)(BM * BN)), part((size_t)BM), rows((size_t)BM, 0.f);
    const float zero = 0.f;
    const int64_t r0 = pid * BM;
    for (int64_t c0 = 0; c0 < n_valid; c0 += BN) {
      const int64_t sz[2] = {BM, BN}, st[2] = {stride_m, stride_n};
      const int64_t dims[2] = {mask_dim(r0, BM, M), mask_dim(c0, BN, n_valid)};
      orc_block_load(x, 4, 2, sz, st, r0 * stride_m + c0 * stride_n, dims, &zero, blk.data());
      std::fill(part.begin(), part.end(), 0.f);
      for (int64_t j = 0; j < BN; ++j)
        for (int64_t i = 0; i < BM; ++i) part[(size_t)i] = blk[(size_t)(i * BN + j)] + part[(size_t)i];
      for (int64_t i = 0; i < BM; ++i) rows[(size_t)i] = rows[(size_t)i] + part[(size_t)i];
    }
    const int64_t one = 1;
    const int64_t dim = mask_dim(r0, BM, M);
    orc_block_store(out, 4, 1, &BM, &one, r0, &dim, rows.data());
  } ORC_END_LOOP;
}

// Scalar total of n values: one program, lane accumulators over blocks of
// `block` (masked, other = 0), then a left-to-right fold into a rank-0 tensor
// (reducesum_scalar.mlir:21-31) and a scalar store.
void orc_reduce_all(const float *x, float *out, int64_t n, int64_t block) {
  std::vector<float> acc((size_t)block, 0.f), b((size_t)block);
  const float zero = 0.f;
  const int64_t one = 1;
  for (int64_t off = 0; off < n; off += block) {
    const int64_t dim = mask_dim(off, block, n);
    orc_block_load(x, 4, 1, &block, &one, off, &dim, &zero, b.data());
    for (int64_t l = 0; l < block; ++l) acc[(size_t)l] = acc[(size_t)l] + b[(size_t)l];
  }
  float s = 0.f;
  for (int64_t l = 0; l < block; ++l) s = acc[(size_t)l] + s;
  out[0] = s;
}

int orc_max_threads(void) {
  unsigned n = std::thread::hardware_concurrency();
  return n > 0 ? (int)n : 1;
}

}  // extern "C"

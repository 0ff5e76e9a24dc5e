// One-program-per-row kernels: fused softmax and LayerNorm forward.
//
// Reference lowered forms these replace (paths inside microsoft/triton-shared):
//   softmax    test/Conversion/StructuredToMemref/kernel-02-fused-softmax.mlir:50-90
//              (python/examples/test_softmax.py:8-29)
//   layernorm  test/Conversion/StructuredToMemref/kernel-05-layer-norm-fwd.mlir
//              (python/examples/test_layernorm.py:29-76)
// In the reference every op is a separate scalar loop over a malloc'ed 1024-lane
// buffer and reductions are left-to-right folds (ConversionPatterns.hpp:1203-1440).
// Here a row is read from HBM once, held in registers, reduced with warp
// shuffles plus a shared-memory step across warps, and written once.
#include "tsb_common.cuh"
#include <math.h>

namespace tsb {

// Sum / max over the TPR threads that share a row. TPR is a multiple of 32 and
// rows never share a warp, so warp w of the CTA belongs to row w / (TPR/32).
template <int TPR, bool IS_MAX>
__device__ __forceinline__ float row_reduce(float v, float *smem /* [THREADS/32] */) {
  v = IS_MAX ? warp_max(v) : warp_sum(v);
  if (TPR == 32) return v;
  constexpr int WPR = TPR / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // smem may still be read by the previous reduction
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  const int w0 = (warp / WPR) * WPR;
  float r = smem[w0];
#pragma unroll
  for (int k = 1; k < WPR; ++k) r = IS_MAX ? fmaxf(r, smem[w0 + k]) : r + smem[w0 + k];
  return r;
}

// Sum over the whole CTA with a single barrier; the caller alternates between two
// `smem` buffers so that a buffer is never rewritten while another warp still reads it.
template <int THREADS>
__device__ __forceinline__ float row_reduce2(float v, float *smem /* [THREADS/32] */) {
  v = warp_sum(v);
  if (THREADS == 32) return v;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float r = smem[0];
#pragma unroll
  for (int k = 1; k < THREADS / 32; ++k) r += smem[k];
  return r;
}

// ---------------------------------------------------------------------------
// softmax, fp32
// A row is covered by TPR threads x VPT vectors x 4 lanes >= n_cols.
// ALIGNED: 16-byte vector path (row bases and strides multiples of 4 floats).
template <int TPR, int VPT, int THREADS, bool ALIGNED>
__global__ void __launch_bounds__(THREADS)
softmax_rows_f32_kernel(const float *__restrict__ in, float *__restrict__ out, long long in_stride,
                        long long out_stride, int n_cols, long long row_lo, long long row_hi) {
  constexpr int RPC = THREADS / TPR;  // rows per CTA
  __shared__ float red[THREADS / 32];
  const int t = threadIdx.x % TPR;
  const long long row = row_lo + (long long)blockIdx.x * RPC + threadIdx.x / TPR;
  const bool live = row < row_hi;
  const float *src = in + (live ? row : row_lo) * in_stride;
  float x[VPT][4];
  const float NEG_INF = __uint_as_float(0xff800000u);
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    if (ALIGNED) {
      const int c = (v * TPR + t) * 4;
      if (live && c + 4 <= n_cols) {
        float4 q = __ldg(reinterpret_cast<const float4 *>(src + c));
        x[v][0] = q.x; x[v][1] = q.y; x[v][2] = q.z; x[v][3] = q.w;
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) x[v][k] = (live && c + k < n_cols) ? __ldg(src + c + k) : NEG_INF;
      }
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int c = (v * 4 + k) * TPR + t;
        x[v][k] = (live && c < n_cols) ? __ldg(src + c) : NEG_INF;
      }
    }
  }
  float m = NEG_INF;
#pragma unroll
  for (int v = 0; v < VPT; ++v)
#pragma unroll
    for (int k = 0; k < 4; ++k) m = fmaxf(m, x[v][k]);
  m = row_reduce<TPR, true>(m, red);
  float s = 0.f;
#pragma unroll
  for (int v = 0; v < VPT; ++v)
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      x[v][k] = expf(x[v][k] - m);
      s += x[v][k];
    }
  s = row_reduce<TPR, false>(s, red);
  if (!live) return;
  float *dst = out + row * out_stride;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    if (ALIGNED) {
      const int c = (v * TPR + t) * 4;
      if (c + 4 <= n_cols) {
        *reinterpret_cast<float4 *>(dst + c) =
            make_float4(x[v][0] / s, x[v][1] / s, x[v][2] / s, x[v][3] / s);
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (c + k < n_cols) dst[c + k] = x[v][k] / s;
      }
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int c = (v * 4 + k) * TPR + t;
        if (c < n_cols) dst[c] = x[v][k] / s;
      }
    }
  }
}

template <int TPR, int VPT, int THREADS>
static int launch_softmax(const float *in, float *out, long long is, long long os, int n_cols,
                          long long row_lo, long long row_hi, bool aligned, cudaStream_t s) {
  constexpr int RPC = THREADS / TPR;
  const long long rows = row_hi - row_lo;
  const long long ctas = (rows + RPC - 1) / RPC;
  if (ctas > 0x7fffffffll) return fail(TSB_ERR_UNSUPPORTED, "tsb_softmax_rows: too many rows");
  if (aligned)
    softmax_rows_f32_kernel<TPR, VPT, THREADS, true><<<(unsigned)ctas, THREADS, 0, s>>>(in, out, is, os, n_cols, row_lo, row_hi);
  else
    softmax_rows_f32_kernel<TPR, VPT, THREADS, false><<<(unsigned)ctas, THREADS, 0, s>>>(in, out, is, os, n_cols, row_lo, row_hi);
  TSB_LAUNCH_OK("softmax_rows_f32_kernel");
  return TSB_OK;
}

// ---------------------------------------------------------------------------
// LayerNorm forward. T = __half / __nv_bfloat16 / float in memory, fp32 math.
template <typename T> struct Io;
template <> struct Io<__half> {
  static constexpr int EPV = 8;
  __device__ static float ld(const __half *p) { return __half2float(*p); }
  __device__ static void st(__half *p, float v) { *p = __float2half_rn(v); }
  __device__ static void unpack(const uint4 &q, float f[8]) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&q);
#pragma unroll
    for (int k = 0; k < 4; ++k) { float2 a = __half22float2(h[k]); f[2 * k] = a.x; f[2 * k + 1] = a.y; }
  }
  __device__ static uint4 pack(const float f[8]) {
    uint4 q; __half2 *h = reinterpret_cast<__half2 *>(&q);
#pragma unroll
    for (int k = 0; k < 4; ++k) h[k] = __halves2half2(__float2half_rn(f[2 * k]), __float2half_rn(f[2 * k + 1]));
    return q;
  }
};
template <> struct Io<__nv_bfloat16> {
  static constexpr int EPV = 8;
  __device__ static float ld(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
  __device__ static void st(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }
  __device__ static void unpack(const uint4 &q, float f[8]) {
    const unsigned *u = reinterpret_cast<const unsigned *>(&q);
#pragma unroll
    for (int k = 0; k < 4; ++k) { f[2 * k] = __uint_as_float(u[k] << 16); f[2 * k + 1] = __uint_as_float(u[k] & 0xffff0000u); }
  }
  __device__ static uint4 pack(const float f[8]) {
    uint4 q; __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&q);
#pragma unroll
    for (int k = 0; k < 4; ++k) h[k] = __halves2bfloat162(__float2bfloat16_rn(f[2 * k]), __float2bfloat16_rn(f[2 * k + 1]));
    return q;
  }
};
template <> struct Io<float> {
  static constexpr int EPV = 4;
  __device__ static float ld(const float *p) { return *p; }
  __device__ static void st(float *p, float v) { *p = v; }
  __device__ static void unpack(const uint4 &q, float f[4]) {
    f[0] = __uint_as_float(q.x); f[1] = __uint_as_float(q.y); f[2] = __uint_as_float(q.z); f[3] = __uint_as_float(q.w);
  }
  __device__ static uint4 pack(const float f[4]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
};

// Persistent CTAs: weight and bias are loaded once per CTA and kept (packed, in
// their memory type) in registers while the CTA walks rows blockIdx.x,
// blockIdx.x + gridDim.x, ...  A row is covered by THREADS x VPT 16-byte vectors.
// Element k of vector v of thread t is column
//   ALIGNED : (v*THREADS + t)*EPV + k   (one 16-byte load per vector)
//   otherwise: (v*EPV + k)*THREADS + t   (scalar loads, still coalesced)
template <typename T, int THREADS, int VPT, bool ALIGNED>
struct RowTile {
  static constexpr int EPV = Io<T>::EPV;
  __device__ static __forceinline__ int col(int v, int k, int t) {
    return ALIGNED ? (v * THREADS + t) * EPV + k : (v * EPV + k) * THREADS + t;
  }
  // shared-memory slot of vector v of thread t (16 bytes each, conflict-free for a warp)
  __device__ static __forceinline__ void put(T *base, int v, int t, const uint4 &q) {
    reinterpret_cast<uint4 *>(base)[v * THREADS + t] = q;
  }
  __device__ static __forceinline__ uint4 get(const T *base, int v, int t) {
    return reinterpret_cast<const uint4 *>(base)[v * THREADS + t];
  }
  __device__ static __forceinline__ void load(const T *src, int n_cols, int t, uint4 q[VPT]) {
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      if (ALIGNED && col(v, EPV - 1, t) < n_cols) {
        q[v] = __ldcs(reinterpret_cast<const uint4 *>(src + col(v, 0, t)));
      } else {
        float f[EPV];
#pragma unroll
        for (int k = 0; k < EPV; ++k) f[k] = col(v, k, t) < n_cols ? Io<T>::ld(src + col(v, k, t)) : 0.f;
        q[v] = Io<T>::pack(f);  // exact: values are already of type T
      }
    }
  }
};

// Weight and bias are read once per CTA.  WB_REGS: they stay in registers in their memory
// type (one 16-byte vector per row vector, converted on use), so the kernel needs no shared
// memory beyond the reduction exchange and its occupancy is set by registers alone.  Otherwise
// (rows too wide for that) they are staged in shared memory, again in their memory type.
// The row is expanded to fp32 registers once, and the next row's 16-byte loads are issued
// before the current row is reduced, so that a CTA always has a full row in flight.  The kernel
// is close to issue-bound, so every per-element instruction counts: masks are evaluated per
// 16-byte vector, not per element.  Products and sums are rounded separately (no contraction),
// as in the reference's lowering.
// resident CTAs per SM the kernel is compiled for (bounds the registers per thread)
constexpr int ln_min_ctas(int threads, int vpt, bool wb_regs) {
  return threads <= 128 ? 1024 / threads
                        : (threads == 256 ? (wb_regs && vpt >= 4 ? 2 : 3) : (threads == 512 ? (vpt >= 4 ? 1 : 2) : 1));
}

template <typename T, int THREADS, int VPT, bool ALIGNED, bool WB_REGS>
__global__ void __launch_bounds__(THREADS, ln_min_ctas(THREADS, VPT, WB_REGS))
layernorm_fwd_kernel(const T *__restrict__ X, T *__restrict__ Y, const T *__restrict__ W,
                     const T *__restrict__ B, float *__restrict__ Mean, float *__restrict__ Rstd,
                     long long xs, long long ys, int n_cols, float eps, long long row_lo,
                     long long row_hi) {
  using Tile = RowTile<T, THREADS, VPT, ALIGNED>;
  constexpr int EPV = Io<T>::EPV;
  extern __shared__ __align__(16) unsigned char ln_smem[];
  T *sw = reinterpret_cast<T *>(ln_smem);
  T *sb = sw + THREADS * VPT * EPV;
  // two exchange buffers, used alternately, so that one barrier per reduction suffices:
  // buffer 0 is next written a full reduction (and its barrier) after its last read
  __shared__ float red[2][THREADS / 32];
  const int t = threadIdx.x;
  grid_dependency_wait();
  grid_launch_dependents();  // all CTAs of this launch are resident: successors only take freed slots
  // the first row's loads go out before weight and bias, so the latencies overlap
  long long row = row_lo + blockIdx.x;
  uint4 xq[VPT];
  if (row < row_hi) Tile::load(X + row * xs, n_cols, t, xq);
  uint4 wq[WB_REGS ? VPT : 1], bq[WB_REGS ? VPT : 1];
  if (WB_REGS) {
    Tile::load(W, n_cols, t, wq);
    Tile::load(B, n_cols, t, bq);
  } else {
    uint4 q[VPT];
    Tile::load(W, n_cols, t, q);
#pragma unroll
    for (int v = 0; v < VPT; ++v) Tile::put(sw, v, t, q[v]);
    Tile::load(B, n_cols, t, q);
#pragma unroll
    for (int v = 0; v < VPT; ++v) Tile::put(sb, v, t, q[v]);
    // each thread reads back only the slots it wrote: no barrier needed
  }
  const float fn = (float)n_cols;
  for (; row < row_hi; row += gridDim.x) {
    float x[VPT][EPV];
#pragma unroll
    for (int v = 0; v < VPT; ++v) Io<T>::unpack(xq[v], x[v]);
    const long long next = row + gridDim.x;
    if (next < row_hi) Tile::load(X + next * xs, n_cols, t, xq);  // in flight during the reductions
    // four independent accumulators per thread keep the add chains short
    float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int v = 0; v < VPT; ++v)
#pragma unroll
      for (int k = 0; k < EPV; ++k) s4[k & 3] += x[v][k];  // lanes >= n_cols hold 0
    const float s = row_reduce2<THREADS>((s4[0] + s4[1]) + (s4[2] + s4[3]), red[0]);
    const float mean = s / fn;
    float q4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      if (Tile::col(v, EPV - 1, t) < n_cols) {
#pragma unroll
        for (int k = 0; k < EPV; ++k) {
          x[v][k] = x[v][k] - mean;  // kept: the output pass starts from the centred value
          q4[k & 3] += x[v][k] * x[v][k];
        }
      } else {
#pragma unroll
        for (int k = 0; k < EPV; ++k) {
          x[v][k] = (Tile::col(v, k, t) < n_cols) ? x[v][k] - mean : 0.f;
          q4[k & 3] += x[v][k] * x[v][k];
        }
      }
    }
    const float q = row_reduce2<THREADS>((q4[0] + q4[1]) + (q4[2] + q4[3]), red[1]);
    const float var = q / fn;
    const float rstd = 1.0f / sqrtf(var + eps);
    if (t == 0) {
      if (Mean) Mean[row] = mean;
      if (Rstd) Rstd[row] = rstd;
    }
    T *dst = Y + row * ys;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      float w[EPV], b[EPV], y[EPV];
      Io<T>::unpack(WB_REGS ? wq[v] : Tile::get(sw, v, t), w);
      Io<T>::unpack(WB_REGS ? bq[v] : Tile::get(sb, v, t), b);
      // x already holds x - mean: ((x - mean) * rstd) * w + b, one rounding per op
#pragma unroll
      for (int k = 0; k < EPV; ++k) y[k] = (x[v][k] * rstd) * w[k] + b[k];
      if (ALIGNED && Tile::col(v, EPV - 1, t) < n_cols) {
        __stcs(reinterpret_cast<uint4 *>(dst + Tile::col(v, 0, t)), Io<T>::pack(y));
      } else {
#pragma unroll
        for (int k = 0; k < EPV; ++k)
          if (Tile::col(v, k, t) < n_cols) Io<T>::st(dst + Tile::col(v, k, t), y[k]);
      }
    }
  }
}

template <typename T, int THREADS, int VPT, bool WB_REGS>
static int launch_ln(const void *x, void *y, const void *w, const void *b, float *mean, float *rstd,
                     long long xs, long long ys, int n_cols, float eps, long long row_lo,
                     long long row_hi, bool aligned, cudaStream_t s) {
  const long long rows = row_hi - row_lo;
  constexpr int SMEM = WB_REGS ? 0 : 2 * THREADS * VPT * 16;  // weight + bias in their memory type
  auto kt = layernorm_fwd_kernel<T, THREADS, VPT, true, WB_REGS>;
  auto kf = layernorm_fwd_kernel<T, THREADS, VPT, false, WB_REGS>;
  static SmemLimit lim_t, lim_f;
  static int per_sm_cache[64][2];
  TSB_CUDA_OK(allow_dynamic_smem(kt, SMEM, lim_t));
  TSB_CUDA_OK(allow_dynamic_smem(kf, SMEM, lim_f));
  const int dev = device_slot();
  int per_sm = per_sm_cache[dev][aligned ? 1 : 0];
  if (per_sm == 0) {
    if (aligned) {
      TSB_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kt, THREADS, SMEM));
    } else {
      TSB_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kf, THREADS, SMEM));
    }
    if (per_sm < 1) per_sm = 1;
    per_sm_cache[dev][aligned ? 1 : 0] = per_sm;
  }
  // all resident CTAs, so that every SM carries the same number of them
  long long ctas = (long long)sm_count() * per_sm;
  if (ctas > rows) ctas = rows;
  TSB_CUDA_OK(launch_pdl(aligned ? kt : kf, dim3((unsigned)ctas), dim3(THREADS), (size_t)SMEM, s, (const T *)x, (T *)y,
                         (const T *)w, (const T *)b, mean, rstd, xs, ys, n_cols, eps, row_lo, row_hi));
  return TSB_OK;
}

template <typename T>
static int dispatch_ln(const void *x, void *y, const void *w, const void *b, float *mean, float *rstd,
                       long long xs, long long ys, long long n_cols, float eps, long long row_lo,
                       long long row_hi, cudaStream_t s) {
  constexpr int EPV = Io<T>::EPV;
  const long long vb = 16;
  const bool aligned = ((uintptr_t)x % vb) == 0 && ((uintptr_t)y % vb) == 0 && ((uintptr_t)w % vb) == 0 &&
                       ((uintptr_t)b % vb) == 0 && xs % EPV == 0 && ys % EPV == 0;
  const long long vecs = (n_cols + EPV - 1) / EPV;  // 16-byte vectors per row
  const int n = (int)n_cols;
#define TSB_LN(THREADS, VPT, WB_REGS) \
  return launch_ln<T, THREADS, VPT, WB_REGS>(x, y, w, b, mean, rstd, xs, ys, n, eps, row_lo, row_hi, aligned, s)
  if (vecs <= 32) TSB_LN(32, 1, true);
  if (vecs <= 64) TSB_LN(64, 1, true);
  if (vecs <= 128) TSB_LN(128, 1, true);
  if (vecs <= 256) TSB_LN(256, 1, true);
  if (vecs <= 512) TSB_LN(256, 2, true);
  // four vectors per thread: weight and bias in shared memory in their memory type (2 * 16 bytes per
  // vector); measured faster than twice the threads with two vectors each and the weights in registers
  if (vecs <= 1024) TSB_LN(256, 4, false);
  if (vecs <= 2048) TSB_LN(512, 4, false);
  if (vecs <= 4096) TSB_LN(1024, 4, false);
#undef TSB_LN
  return fail(TSB_ERR_UNSUPPORTED, "tsb_layernorm_fwd: rows of %lld elements exceed the on-chip limit (%d)",
              n_cols, 4096 * EPV);
}

}  // namespace tsb

using namespace tsb;

extern "C" int tsb_softmax_rows(const void *in, void *out, int32_t dtype, int64_t in_row_stride,
                                int64_t out_row_stride, int64_t n_cols, int64_t block,
                                int64_t row_lo, int64_t row_hi, void *stream) {
  if (!in || !out) return fail(TSB_ERR_INVALID, "tsb_softmax_rows: null pointer");
  if (dtype != TSB_F32) return fail(TSB_ERR_UNSUPPORTED, "tsb_softmax_rows: only fp32 rows are implemented (dtype %d)", dtype);
  if (row_lo < 0 || row_hi < row_lo) return fail(TSB_ERR_INVALID, "tsb_softmax_rows: bad row range");
  if (n_cols < 0 || block <= 0) return fail(TSB_ERR_INVALID, "tsb_softmax_rows: bad n_cols/block");
  if (row_hi == row_lo) return TSB_OK;
  // Lanes >= min(n_cols, block) hold -inf and contribute exp(-inf) = 0.
  const long long n = n_cols < block ? n_cols : block;
  if (n == 0) return TSB_OK;
  const bool aligned = ((uintptr_t)in % 16) == 0 && ((uintptr_t)out % 16) == 0 &&
                       in_row_stride % 4 == 0 && out_row_stride % 4 == 0;
  cudaStream_t s = (cudaStream_t)stream;
  const float *i = (const float *)in;
  float *o = (float *)out;
#define TSB_SM(TPR, VPT, THREADS) \
  return launch_softmax<TPR, VPT, THREADS>(i, o, in_row_stride, out_row_stride, (int)n, row_lo, row_hi, aligned, s)
  if (n <= 128) TSB_SM(32, 1, 256);
  if (n <= 256) TSB_SM(32, 2, 256);
  if (n <= 512) TSB_SM(32, 4, 256);
  if (n <= 1024) TSB_SM(32, 8, 256);
  if (n <= 2048) TSB_SM(128, 4, 256);
  if (n <= 4096) TSB_SM(256, 4, 256);
  if (n <= 8192) TSB_SM(256, 8, 256);
  if (n <= 16384) TSB_SM(512, 8, 512);
  if (n <= 32768) TSB_SM(1024, 8, 1024);
#undef TSB_SM
  return fail(TSB_ERR_UNSUPPORTED, "tsb_softmax_rows: rows of %lld columns exceed the register-resident limit (32768)", n);
}

extern "C" int tsb_layernorm_fwd(const void *x, void *y, const void *w, const void *b, float *mean,
                                 float *rstd, int32_t io_dtype, int64_t x_row_stride,
                                 int64_t y_row_stride, int64_t n_cols, float eps, int64_t row_lo,
                                 int64_t row_hi, void *stream) {
  if (!x || !y || !w || !b) return fail(TSB_ERR_INVALID, "tsb_layernorm_fwd: null pointer");
  if (row_lo < 0 || row_hi < row_lo || n_cols <= 0) return fail(TSB_ERR_INVALID, "tsb_layernorm_fwd: bad range");
  if (row_hi == row_lo) return TSB_OK;
  cudaStream_t s = (cudaStream_t)stream;
  switch (io_dtype) {
    case TSB_F16: return dispatch_ln<__half>(x, y, w, b, mean, rstd, x_row_stride, y_row_stride, n_cols, eps, row_lo, row_hi, s);
    case TSB_BF16: return dispatch_ln<__nv_bfloat16>(x, y, w, b, mean, rstd, x_row_stride, y_row_stride, n_cols, eps, row_lo, row_hi, s);
    case TSB_F32: return dispatch_ln<float>(x, y, w, b, mean, rstd, x_row_stride, y_row_stride, n_cols, eps, row_lo, row_hi, s);
  }
  return fail(TSB_ERR_UNSUPPORTED, "tsb_layernorm_fwd: dtype %d", io_dtype);
}

// Strided masked 2-D sums along axis 1, and the full 1-D sum.
//
// Reference lowered form this replaces (paths inside microsoft/triton-shared):
//   masked 2-D block load   test/Conversion/StructuredToMemref/masked_ldst_2d.mlir:76-99
//   sum over axis 1         test/Conversion/StructuredToMemref/reducesum_512_256_f32_axis1.mlir
//                           (transpose + linalg.reduce dims=[0], ConversionPatterns.hpp:1343-1407)
//   scalar sum              test/Conversion/StructuredToMemref/reducesum_scalar.mlir:21-31
// The CPU backend copies each ragged block element by element
// (CRunnerUtils.cpp:58-113) and folds left to right on one thread.
#include "tsb_common.cuh"
#include <cooperative_groups.h>

namespace tsb {

// ---- kept dim contiguous (stride_m == 1): "column sums of a row-major matrix" ----
// CTA = 8 warps and a tile of 128 consecutive rows i. With VEC4 a lane owns rows
// 4*lane..4*lane+3 of the tile and issues one 16-byte load per j; otherwise it
// owns rows lane, lane+32, lane+64, lane+96 (scalar loads, still coalesced).
// The 8 warps take interleaved j. blockIdx.y selects a slice of j (a "split");
// partial sums of split s go to dst[s*dst_stride_split + i] (straight to the
// output when there is one split).
constexpr int RC_WARPS = 8;
constexpr int RC_UNROLL = 8;
constexpr int RC_TILE = 128;

// CLUSTER: the CTAs that share a row tile (blockIdx.y = split) form one thread-block cluster.
// Each leaves its 128 partial sums in its own shared memory; after a cluster barrier the CTA of
// rank 0 adds them in split order through distributed shared memory and writes the row sums, so
// that the whole reduction is one launch with no global scratch and a fixed order of additions.
template <bool VEC4, bool CLUSTER>
__global__ void __launch_bounds__(RC_WARPS * 32)
reduce_rows_contig_m_kernel(const float *__restrict__ x, float *__restrict__ dst,
                            long long dst_stride_i, long long dst_stride_split, long long stride_n,
                            long long n_valid, long long row_lo, long long row_hi, int j_per_split) {
  __shared__ float red[RC_WARPS][RC_TILE];
  __shared__ float tile_sum[RC_TILE];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long tile0 = row_lo + (long long)blockIdx.x * RC_TILE;
  const long long j_lo = (long long)blockIdx.y * j_per_split;
  long long j_hi = j_lo + j_per_split;
  if (j_hi > n_valid) j_hi = n_valid;
  grid_dependency_wait();
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  if (VEC4 && tile0 + RC_TILE <= row_hi) {
    const float *p = x + tile0 + lane * 4;
    long long j = j_lo + warp;
    // RC_UNROLL independent 16-byte loads in flight per thread
    for (; j + (RC_UNROLL - 1) * RC_WARPS < j_hi; j += RC_UNROLL * RC_WARPS) {
      float4 q[RC_UNROLL];
#pragma unroll
      for (int u = 0; u < RC_UNROLL; ++u)
        q[u] = __ldcs(reinterpret_cast<const float4 *>(p + (j + u * RC_WARPS) * stride_n));
#pragma unroll
      for (int u = 0; u < RC_UNROLL; ++u) {
        acc[0] += q[u].x; acc[1] += q[u].y; acc[2] += q[u].z; acc[3] += q[u].w;
      }
    }
    for (; j < j_hi; j += RC_WARPS) {
      float4 q = __ldcs(reinterpret_cast<const float4 *>(p + j * stride_n));
      acc[0] += q.x; acc[1] += q.y; acc[2] += q.z; acc[3] += q.w;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) red[warp][lane * 4 + k] = acc[k];
  } else {
    for (long long j = j_lo + warp; j < j_hi; j += RC_WARPS)
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const long long i = tile0 + lane + 32 * k;
        if (i < row_hi) acc[k] += __ldg(x + i + j * stride_n);
      }
#pragma unroll
    for (int k = 0; k < 4; ++k) red[warp][lane + 32 * k] = acc[k];
  }
  grid_launch_dependents();
  __syncthreads();
  // 128 row sums per CTA, combined over the 8 warps in a fixed order
  float s = 0.f;
  if (threadIdx.x < RC_TILE) {
    const int r = threadIdx.x;
    s = red[0][r];
#pragma unroll
    for (int w = 1; w < RC_WARPS; ++w) s += red[w][r];
  }
  if (CLUSTER) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    if (threadIdx.x < RC_TILE) tile_sum[threadIdx.x] = s;
    cluster.sync();  // every split's partial sums are in place
    if (cluster.block_rank() == 0 && threadIdx.x < RC_TILE) {
      const unsigned n = cluster.num_blocks();
      float t = tile_sum[threadIdx.x];
      for (unsigned k = 1; k < n; ++k) t += cluster.map_shared_rank(tile_sum, k)[threadIdx.x];  // split order
      const long long i = tile0 + threadIdx.x;
      if (i < row_hi) dst[(i - row_lo) * dst_stride_i] = t;
    }
    cluster.sync();  // no CTA leaves while its shared memory may still be read
  } else if (threadIdx.x < RC_TILE) {
    const long long i = tile0 + threadIdx.x;
    if (i < row_hi) dst[(i - row_lo) * dst_stride_i + (long long)blockIdx.y * dst_stride_split] = s;
  }
}

// Sum the per-split partials: out[i] = sum_s part[s*n_rows + i], s ascending.
__global__ void reduce_rows_finalize_kernel(const float *__restrict__ part, float *__restrict__ out,
                                            long long out_stride, long long n_rows, int splits,
                                            long long row_lo) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_rows) return;
  float s = 0.f;
  for (int k = 0; k < splits; ++k) s += part[(long long)k * n_rows + i];
  out[(row_lo + i) * out_stride] = s;
}

// ---- reduced dim contiguous (stride_n == 1): one warp per row -----------------
__global__ void __launch_bounds__(256)
reduce_rows_contig_n_kernel(const float *__restrict__ x, float *__restrict__ out, long long stride_m,
                            long long out_stride, long long n_valid, long long row_lo,
                            long long row_hi, int vec_ok) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long i = row_lo + (long long)blockIdx.x * 8 + warp;
  if (i >= row_hi) return;
  const float *p = x + i * stride_m;
  float s = 0.f;
  if (vec_ok) {
    const long long nv = n_valid / 4;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    for (long long v = lane; v < nv; v += 32) {
      float4 q = __ldg(reinterpret_cast<const float4 *>(p) + v);
      a0 += q.x; a1 += q.y; a2 += q.z; a3 += q.w;
    }
    s = (a0 + a1) + (a2 + a3);
    for (long long j = nv * 4 + lane; j < n_valid; j += 32) s += __ldg(p + j);
  } else {
    for (long long j = lane; j < n_valid; j += 32) s += __ldg(p + j);
  }
  s = warp_sum(s);
  if (lane == 0) out[i * out_stride] = s;
}

// ---- arbitrary strides: one thread per row ------------------------------------
__global__ void reduce_rows_generic_kernel(const float *__restrict__ x, float *__restrict__ out,
                                           long long stride_m, long long stride_n,
                                           long long out_stride, long long n_valid,
                                           long long row_lo, long long row_hi) {
  const long long i = row_lo + (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= row_hi) return;
  float s = 0.f;
  for (long long j = 0; j < n_valid; ++j) s += __ldg(x + i * stride_m + j * stride_n);
  out[i * out_stride] = s;
}

// ---- full sum: one CTA, fixed order --------------------------------------------
__global__ void __launch_bounds__(1024)
reduce_all_kernel(const float *__restrict__ x, float *__restrict__ out, long long n, long long stride) {
  __shared__ float red[32];
  grid_dependency_wait();
  grid_launch_dependents();
  float s = 0.f;
  for (long long i = threadIdx.x; i < n; i += 1024) s += __ldg(x + i * stride);
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = red[threadIdx.x];
    v = warp_sum(v);
    if (threadIdx.x == 0) out[0] = v;
  }
}

struct ContigMPlan {
  long long i_tiles;
  int splits;
  int j_per_split;
  bool cluster;  // the splits of a row tile form one cluster (no scratch, one launch)
};

constexpr int RC_MAX_CLUSTER = 16;  // 8 is the portable limit; 16 is opted into per device

// Largest cluster (splits per row tile) this device schedules for the kernel: 16 where the
// non-portable size is available, else the portable 8.  Asked once per device.
static int max_cluster_splits() {
  static int cached[64];
  const int dev = device_slot();
  if (cached[dev]) return cached[dev];
  int best = 8;
  auto kern = reduce_rows_contig_m_kernel<true, true>;
  auto kern2 = reduce_rows_contig_m_kernel<false, true>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess &&
      cudaFuncSetAttribute(kern2, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1, RC_MAX_CLUSTER, 1);
    cfg.blockDim = dim3(RC_WARPS * 32, 1, 1);
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 1;
    at[0].val.clusterDim.y = RC_MAX_CLUSTER;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) == cudaSuccess && n > 0) best = RC_MAX_CLUSTER;
  }
  (void)cudaGetLastError();  // a refused query is an answer, not an error of the caller
  cached[dev] = best;
  return best;
}

// Depends on the problem shape only, so that the scratch size a caller asked
// for earlier always matches the launch.
static ContigMPlan plan_contig_m(long long n_rows, long long n_valid) {
  ContigMPlan p;
  p.i_tiles = (n_rows + RC_TILE - 1) / RC_TILE;
  // enough CTAs for two full waves of 8 CTAs per SM; each split keeps >= 64 j
  long long want = (2ll * 8 * sm_count() + p.i_tiles - 1) / p.i_tiles;
  const long long max_splits = (n_valid + 63) / 64;
  if (want > max_splits) want = max_splits;
  if (want > 1024) want = 1024;
  if (want < 1) want = 1;
  // With enough row tiles, 16 splits per tile already put four or more CTAs on every SM: then
  // the splits are combined inside a cluster.  Fewer tiles need more splits than a cluster holds
  // and go through partial sums in scratch memory.
  p.cluster = want > 1 && want <= 4 * RC_MAX_CLUSTER;
  if (p.cluster) {
    int c = 1;
    const int cmax = max_cluster_splits();
    while (c < want && c < cmax) c *= 2;
    want = c;
  }
  p.j_per_split = (int)((n_valid + want - 1) / want);
  if (p.j_per_split < 1) p.j_per_split = 1;
  p.splits = p.cluster ? (int)want : (int)((n_valid + p.j_per_split - 1) / p.j_per_split);
  if (p.splits < 1) p.splits = 1;
  return p;
}

template <bool VEC4>
static int launch_contig_m_cluster(const ContigMPlan &p, const float *x, float *out, long long out_stride,
                                   long long stride_n, long long n_valid, long long row_lo, long long row_hi,
                                   cudaStream_t s) {
  auto kern = reduce_rows_contig_m_kernel<VEC4, true>;  // cluster sizes above 8: see max_cluster_splits()
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)p.i_tiles, (unsigned)p.splits, 1);
  cfg.blockDim = dim3(RC_WARPS * 32, 1, 1);
  cfg.stream = s;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 1;
  at[0].val.clusterDim.y = (unsigned)p.splits;
  at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  TSB_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, x, out + row_lo * out_stride, out_stride, 0ll, stride_n, n_valid, row_lo,
                                 row_hi, p.j_per_split));
  return TSB_OK;
}

}  // namespace tsb

using namespace tsb;

extern "C" int64_t tsb_reduce_rows_scratch_bytes(int64_t n_rows, int64_t n_valid, int64_t stride_m,
                                                 int64_t stride_n) {
  (void)stride_n;
  if (n_rows <= 0 || n_valid <= 0 || stride_m != 1) return 0;
  ContigMPlan p = plan_contig_m(n_rows, n_valid);
  return (p.splits > 1 && !p.cluster) ? (int64_t)p.splits * n_rows * (int64_t)sizeof(float) : 0;
}

extern "C" int tsb_reduce_rows(const float *x, float *out, int64_t stride_m, int64_t stride_n,
                               int64_t out_stride, int64_t n_valid, int64_t row_lo, int64_t row_hi,
                               void *scratch, void *stream) {
  if (!x || !out) return fail(TSB_ERR_INVALID, "tsb_reduce_rows: null pointer");
  if (row_lo < 0 || row_hi < row_lo || n_valid < 0) return fail(TSB_ERR_INVALID, "tsb_reduce_rows: bad range");
  const long long n_rows = row_hi - row_lo;
  if (n_rows == 0) return TSB_OK;
  cudaStream_t s = (cudaStream_t)stream;
  if (stride_m == 1 && n_valid > 0) {
    const ContigMPlan p = plan_contig_m(n_rows, n_valid);
    const bool vec4 = ((uintptr_t)(x + row_lo) % 16) == 0 && stride_n % 4 == 0;
    if (p.cluster)
      return vec4 ? launch_contig_m_cluster<true>(p, x, out, out_stride, stride_n, n_valid, row_lo, row_hi, s)
                  : launch_contig_m_cluster<false>(p, x, out, out_stride, stride_n, n_valid, row_lo, row_hi, s);
    if (p.splits > 1 && !scratch)
      return fail(TSB_ERR_INVALID, "tsb_reduce_rows: %lld bytes of scratch required, got NULL",
                  (long long)p.splits * n_rows * (long long)sizeof(float));
    dim3 grid((unsigned)p.i_tiles, (unsigned)p.splits);
    float *dst = p.splits > 1 ? (float *)scratch : out + row_lo * out_stride;
    const long long dsi = p.splits > 1 ? 1 : out_stride;
    const long long dss = p.splits > 1 ? n_rows : 0;
    if (vec4)
      reduce_rows_contig_m_kernel<true, false><<<grid, RC_WARPS * 32, 0, s>>>(x, dst, dsi, dss, stride_n, n_valid, row_lo, row_hi, p.j_per_split);
    else
      reduce_rows_contig_m_kernel<false, false><<<grid, RC_WARPS * 32, 0, s>>>(x, dst, dsi, dss, stride_n, n_valid, row_lo, row_hi, p.j_per_split);
    TSB_LAUNCH_OK("reduce_rows_contig_m_kernel");
    if (p.splits > 1) {
      reduce_rows_finalize_kernel<<<(unsigned)((n_rows + 255) / 256), 256, 0, s>>>(
          (const float *)scratch, out, out_stride, n_rows, p.splits, row_lo);
      TSB_LAUNCH_OK("reduce_rows_finalize_kernel");
    }
    return TSB_OK;
  }
  if (stride_n == 1 || n_valid == 0) {
    const int vec_ok = ((uintptr_t)x % 16) == 0 && stride_m % 4 == 0;
    reduce_rows_contig_n_kernel<<<(unsigned)((n_rows + 7) / 8), 256, 0, s>>>(x, out, stride_m, out_stride, n_valid, row_lo, row_hi, vec_ok);
    TSB_LAUNCH_OK("reduce_rows_contig_n_kernel");
    return TSB_OK;
  }
  reduce_rows_generic_kernel<<<(unsigned)((n_rows + 127) / 128), 128, 0, s>>>(x, out, stride_m, stride_n, out_stride, n_valid, row_lo, row_hi);
  TSB_LAUNCH_OK("reduce_rows_generic_kernel");
  return TSB_OK;
}

extern "C" int tsb_reduce_all(const float *x, float *out, int64_t n, int64_t stride, void *stream) {
  if (!x || !out) return fail(TSB_ERR_INVALID, "tsb_reduce_all: null pointer");
  if (n < 0) return fail(TSB_ERR_INVALID, "tsb_reduce_all: negative length");
  TSB_CUDA_OK(launch_pdl(reduce_all_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream, x, out, (long long)n,
                         (long long)stride));
  return TSB_OK;
}

// ---------------------------------------------------------------------------
// Allocation-free variant of tsb_reduce_rows.
//
// tsb_reduce_rows wants the caller to hand it device scratch for the per-split
// partial sums.  Some hosts cannot produce such a buffer at the point of the
// call: a launcher written in plain C or ctypes with no device allocator of its
// own, a process whose whole device memory is already carved up by another
// framework's arena, or a latency-critical loop that must not risk the implicit
// device-wide synchronisation of cudaMalloc/cudaFree.  For them the partials live
// in a fixed array inside this library's device image.
//
// Facts a user must know:
//  * The array is TSB_REDUCE_STATIC_SCRATCH_BYTES (1 MiB) of device memory per GPU
//    that loads the library, held until the process exits.
//  * Calls whose partials do not fit are refused with TSB_ERR_UNSUPPORTED; nothing
//    is allocated behind the caller's back (no cudaMalloc, cudaFree, or any
//    allocating library routine is reached from this entry point).
//  * Every call on a device shares the one array and finds in it whatever the
//    previous call left.  Nothing needs clearing: the combine step only reads
//    partials that the first step of the same call has written.  Two calls that
//    overlap on the GPU (different streams, or different host threads) race on
//    the array; issue them on one stream or order them with events.
//  * The first call on each device resolves the array's device address
//    (cudaGetSymbolAddress, with that device current) and caches it; make that
//    first call before starting any stream capture.
static __device__ __align__(256) float g_reduce_static_scratch[TSB_REDUCE_STATIC_SCRATCH_BYTES / sizeof(float)];

namespace tsb {
// In host code the array's name is only a handle for the runtime, not a device
// address, so the address handed to the kernels is looked up once per device.
static int reduce_static_scratch(float **out) {
  static float *per_device[64] = {nullptr};
  int dev = -1;
  TSB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(TSB_ERR_UNSUPPORTED, "tsb_reduce_rows_static: device ordinal %d", dev);
  float *p = __atomic_load_n(&per_device[dev], __ATOMIC_ACQUIRE);
  if (!p) {
    void *addr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&addr, g_reduce_static_scratch);
    if (e != cudaSuccess || !addr)
      return fail(TSB_ERR_CUDA, "tsb_reduce_rows_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    p = static_cast<float *>(addr);
    __atomic_store_n(&per_device[dev], p, __ATOMIC_RELEASE);  // racing first calls store the same value
  }
  *out = p;
  return TSB_OK;
}
}  // namespace tsb

extern "C" int tsb_reduce_rows_static(const float *x, float *out, int64_t stride_m, int64_t stride_n,
                                      int64_t out_stride, int64_t n_valid, int64_t row_lo, int64_t row_hi,
                                      void *stream) {
  if (row_lo < 0 || row_hi < row_lo || n_valid < 0) return fail(TSB_ERR_INVALID, "tsb_reduce_rows_static: bad range");
  const int64_t need = tsb_reduce_rows_scratch_bytes(row_hi - row_lo, n_valid, stride_m, stride_n);
  if (need > (int64_t)TSB_REDUCE_STATIC_SCRATCH_BYTES)
    return fail(TSB_ERR_UNSUPPORTED,
                "tsb_reduce_rows_static: this shape needs %lld bytes of partial sums but the built-in array holds %lld; "
                "use tsb_reduce_rows with caller-provided scratch",
                (long long)need, (long long)TSB_REDUCE_STATIC_SCRATCH_BYTES);
  float *scratch = nullptr;
  if (need > 0) {
    int rc = reduce_static_scratch(&scratch);
    if (rc != TSB_OK) return rc;
  }
  return tsb_reduce_rows(x, out, stride_m, stride_n, out_stride, n_valid, row_lo, row_hi, scratch, stream);
}

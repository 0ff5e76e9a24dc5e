// tt.dot path: C[M,N] = A[M,K] * B[K,N], fp16/bf16 operands, fp32 accumulation.
//
// Reference semantics (paths inside microsoft/triton-shared): per K step the
// lowered kernel loads a zero-filled A block and B block (masked_ldst_2d form),
// runs linalg.matmul from a zero tile with k ascending, adds it to the running
// accumulator (MatmulConverter, ConversionPatterns.hpp:1128-1201) and finally
// truncates once and stores the clipped tile
// (test/Conversion/StructuredToMemref/kernel-03-matrix-multiplication.mlir:157-204).
// The CPU backend executes that as scalar i-j-k loops on one thread.
//
// Two kernels:
//  * gemm_tcgen05_kernel: persistent, warp-specialised.  One thread issues TMA
//    tile loads (cp.async.bulk.tensor, 128-byte swizzle, zero fill outside the
//    tensor = the masked loads' other=0) into a ring of shared-memory stages; one
//    thread issues tcgen05.mma (M=128, N=BLOCK_N, K=16 per instruction) whose fp32
//    accumulator lives in tensor memory, double-buffered so that four epilogue
//    warps can drain tile t (tcgen05.ld -> convert -> global stores clipped to
//    M,N) while tile t+1 is being accumulated.  Programs are walked in pid order
//    through the caller's pid -> tile table, so the kernel author's grouped
//    ordering is what the L2 sees.  No cluster launch and no multicast.
//  * gemm_simt_kernel: plain shared-memory tiled fp32 kernel for everything the
//    tensor path cannot take (row pitches that are not multiples of 16 bytes,
//    block shapes other than 128 x {64..256} x 64k, fp32 operands).
//
// Every wait on an mbarrier is bounded by wall-clock time; on expiry the kernel
// records where it gave up in status[], stops issuing work, drains its
// outstanding copies with a second bounded wait, frees its tensor memory and
// returns.
#include "tsb_tcgen05.cuh"
#include <string.h>

namespace tsb {

// ------------------------------------------------------------------ tensor-core kernel
constexpr int GEMM_THREADS = 192;  // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2-5: epilogue

struct GemmParams {
  void *c;
  long long M, N, K;
  long long scm;                 // C row pitch in elements (unit column stride)
  const int *tile_of_pid;        // (tile_m, tile_n) per program of the full grid
  long long pid_lo, pid_hi;
  int *status;                   // status[0] = failure code, [1] = role, [2] = tile index, [3] = k step
  int block_n;                   // 16..256, multiple of 16 (multiple of 64 when B is MN-major)
  int k_sub;                     // BLOCK_K / 64: stages consumed per K step of the Triton kernel
  int stages;
  int is_bf16;
  int b_mn_major;                // B given as [K,N] with unit stride along N
  int c_vec_ok;                  // 16-byte stores allowed (pitch and base aligned)
  int tmem_cols;                 // allocated tensor-memory columns (power of two >= 2*block_n)
  uint32_t idesc;
};

__device__ __forceinline__ void give_up(const GemmParams &P, volatile int *abort_flag, int role, long long tile, int k) {
  if (atomicCAS((int *)abort_flag, 0, 1) == 0 && P.status) {
    P.status[1] = role;
    P.status[2] = (int)tile;
    P.status[3] = k;
    __threadfence();
    atomicExch(&P.status[0], TSB_ERR_TIMEOUT);
  }
}

__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ GemmParams P) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) unsigned long long bars[2 * 8 + 4];  // full[8], empty[8], tmem_full[2], tmem_empty[2]
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int BN = P.block_n;
  const int S = P.stages;
  const uint32_t b_stage_bytes = (uint32_t)GEMM_BK * BN * 2;
  const uint32_t stage_bytes = A_STAGE_BYTES + b_stage_bytes;
  // tiles need 1024-byte alignment for the 128-byte swizzle pattern
  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  auto full_bar = [&](int s) { return smem_u32(&bars[s]); };
  auto empty_bar = [&](int s) { return smem_u32(&bars[8 + s]); };
  auto tfull_bar = [&](int a) { return smem_u32(&bars[16 + a]); };
  auto tempty_bar = [&](int a) { return smem_u32(&bars[18 + a]); };

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < S; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);  // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_slot), (uint32_t)P.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  const long long n_tiles = P.pid_hi - P.pid_lo;
  const int k_iters = (int)((P.K + GEMM_BK - 1) / GEMM_BK);

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int s = 0;
      uint32_t phase = 0;
      long long issued = 0;
      bool ok = true;
      for (long long t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
        const int tm = P.tile_of_pid[2 * (P.pid_lo + t)], tn = P.tile_of_pid[2 * (P.pid_lo + t) + 1];
        for (int k = 0; k < k_iters; ++k) {
          if (!mbar_wait(empty_bar(s), phase ^ 1u, &abort_flag)) {
            give_up(P, &abort_flag, 0, t, k);
            ok = false;
            break;
          }
          const uint32_t a_dst = smem0 + (uint32_t)s * stage_bytes;
          const uint32_t b_dst = a_dst + A_STAGE_BYTES;
          mbar_expect_tx(full_bar(s), stage_bytes);
          tma_load_2d(a_dst, &map_a, k * GEMM_BK, tm * GEMM_BM, full_bar(s));
          if (P.b_mn_major) {
            // [K,N] row-major: boxes of 64 k-rows x 64 n (128 bytes); chunk c of the tile's N range
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(b_dst + (uint32_t)c * (GEMM_BK * 128), &map_b, tn * BN + c * 64, k * GEMM_BK, full_bar(s));
          } else {
            tma_load_2d(b_dst, &map_b, k * GEMM_BK, tn * BN, full_bar(s));
          }
          ++issued;
          if (++s == S) { s = 0; phase ^= 1u; }
        }
      }
      if (!ok || abort_flag) {
        // drain: every armed stage either completes or the short limit expires
        const long long pending = issued < S ? issued : S;
        int ds = s;
        uint32_t dphase = phase;
        for (long long i = 0; i < pending; ++i) {
          if (--ds < 0) { ds = S - 1; dphase ^= 1u; }
          mbar_wait(full_bar(ds), dphase, &abort_flag, DRAIN_LIMIT_NS);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int s = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (long long t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
        if (k_iters > 0) {
          if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, &abort_flag)) {
            give_up(P, &abort_flag, 1, t, -1);
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
          for (int k = 0; k < k_iters; ++k) {
            if (!mbar_wait(full_bar(s), phase, &abort_flag)) {
              give_up(P, &abort_flag, 1, t, k);
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t a_src = smem0 + (uint32_t)s * stage_bytes;
            const uint32_t b_src = a_src + A_STAGE_BYTES;
#pragma unroll
            for (int kk = 0; kk < GEMM_BK / 16; ++kk) {
              // A, K-major: 8-row groups 1024 bytes apart; 16 elements of K = 32 bytes along the row
              const uint64_t ad = make_smem_desc(a_src + kk * 32, 16, 1024);
              // B, MN-major: 64-column chunks GEMM_BK*128 bytes apart (leading), 8 k-rows = 1024 bytes
              //    K-major : same form as A with N rows
              const uint64_t bd = P.b_mn_major ? make_smem_desc(b_src + kk * 16 * 128, GEMM_BK * 128, 1024)
                                               : make_smem_desc(b_src + kk * 32, 16, 1024);
              umma_f16(d_tmem, ad, bd, P.idesc, (k > 0 || kk > 0) ? 1u : 0u);
            }
            umma_commit(empty_bar(s));  // frees the stage once these MMAs have read it
            if (++s == S) { s = 0; phase ^= 1u; }
          }
          if (ok) umma_commit(tfull_bar(acc));
        }
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ---------------- epilogue: TMEM -> registers -> global ----------------
    const int q = warp & 3;  // tensor-memory lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    for (long long t = blockIdx.x; t < n_tiles; t += gridDim.x) {
      const int tm = P.tile_of_pid[2 * (P.pid_lo + t)], tn = P.tile_of_pid[2 * (P.pid_lo + t) + 1];
      bool have = false;
      if (k_iters > 0) {
        have = mbar_wait(tfull_bar(acc), acc_phase, &abort_flag);
        if (!have) {
          give_up(P, &abort_flag, 2, t, -1);
          break;
        }
        tc_fence_after();
      }
      const long long row = (long long)tm * GEMM_BM + q * 32 + lane;
      const long long col0 = (long long)tn * BN;
      for (int c = 0; c < BN; c += 32) {
        uint32_t v[32];
        if (have) {
          tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c), v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;  // K == 0: the accumulator is the zero tile
        }
        if (row < P.M) {
          unsigned short *crow = reinterpret_cast<unsigned short *>(P.c) + row * P.scm + col0 + c;
          uint32_t packed[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float lo = __uint_as_float(v[2 * i]), hi = __uint_as_float(v[2 * i + 1]);
            if (P.is_bf16) {
              __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
              packed[i] = *reinterpret_cast<uint32_t *>(&h);
            } else {
              __half2 h = __floats2half2_rn(lo, hi);
              packed[i] = *reinterpret_cast<uint32_t *>(&h);
            }
          }
          const long long cols_left = P.N - (col0 + c);
          if (P.c_vec_ok && cols_left >= 32) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              reinterpret_cast<uint4 *>(crow)[i] =
                  make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < cols_left) crow[i] = (unsigned short)(packed[i >> 1] >> ((i & 1) * 16));
          }
        }
      }
      if (have) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(acc));
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)P.tmem_cols);
  }
}

// ------------------------------------------------------------------ SIMT fallback
// 64 x 64 output tile per CTA of 256 threads (4 x 4 outputs each), K stepped by 16.
// Covers arbitrary strides and alignments; products are exact in fp32 for 16-bit inputs.
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }

struct SimtParams {
  const void *a, *b;
  void *c;
  long long M, N, K, sam, sak, sbk, sbn, scm, scn;
  const int *tile_of_pid;
  long long pid_lo, pid_hi;
  int block_m, block_n;
};

template <typename T>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const __grid_constant__ SimtParams P) {
  __shared__ float As[16][64 + 1];
  __shared__ float Bs[16][64 + 1];
  const T *A = (const T *)P.a;
  const T *B = (const T *)P.b;
  T *C = (T *)P.c;
  // blockIdx.x: program (relative to pid_lo); blockIdx.y: 64x64 sub-tile of that program's block
  const long long pid = P.pid_lo + blockIdx.x;
  const int subs_n = (P.block_n + 63) / 64;
  const int sub_m = blockIdx.y / subs_n, sub_n = blockIdx.y % subs_n;
  const long long tile_r0 = (long long)P.tile_of_pid[2 * pid] * P.block_m;
  const long long tile_c0 = (long long)P.tile_of_pid[2 * pid + 1] * P.block_n;
  const long long r0 = tile_r0 + sub_m * 64, c0 = tile_c0 + sub_n * 64;
  const long long r_end = min(min(tile_r0 + P.block_m, P.M), r0 + 64);
  const long long c_end = min(min(tile_c0 + P.block_n, P.N), c0 + 64);
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (long long k0 = 0; k0 < P.K; k0 += 16) {
    for (int e = threadIdx.x; e < 16 * 64; e += 256) {
      const int kk = e & 15, m = e >> 4;
      const long long r = r0 + m, k = k0 + kk;
      As[kk][m] = (r < r_end && k < P.K) ? to_f32<T>(A[r * P.sam + k * P.sak]) : 0.f;
      const int n = e & 63, kb = e >> 6;
      const long long c = c0 + n, k2 = k0 + kb;
      Bs[kb][n] = (c < c_end && k2 < P.K) ? to_f32<T>(B[k2 * P.sbk + c * P.sbn]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = acc[i][j] + a[i] * b[j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long r = r0 + ty * 4 + i, c = c0 + tx * 4 + j;
      if (r < r_end && c < c_end) C[r * P.scm + c * P.scn] = from_f32<T>(acc[i][j]);
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// 2-D map over a row-major [rows, inner] matrix with `pitch` elements between rows.
int make_map(CUtensorMap *m, const void *base, int is_bf16, long long inner, long long rows,
                    long long pitch, int box_inner, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(TSB_ERR_CUDA, "tsb_gemm: cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)pitch * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                  const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(TSB_ERR_CUDA, "tsb_gemm: cuTensorMapEncodeTiled failed with code %d", (int)r);
  return TSB_OK;
}

// 0: not eligible for the tensor-core kernel; 1: B is MN-major ([K,N], unit stride along N);
// 2: B is K-major (unit stride along K).
int tensor_path_mode(const void *a, const void *b, int dtype, long long sam, long long sak,
                            long long sbk, long long sbn, long long scn, int bm, int bn, int bk) {
  if (dtype != TSB_BF16 && dtype != TSB_F16) return 0;
  if (bm != GEMM_BM || bk % GEMM_BK != 0 || bn < 16 || bn > 256 || bn % 16 != 0) return 0;
  if (sak != 1 || scn != 1) return 0;
  if (((uintptr_t)a % 16) || ((uintptr_t)b % 16) || sam % 8) return 0;  // TMA: 16-byte base and pitch
  if (sbn == 1 && sbk % 8 == 0 && bn % 64 == 0) return 1;
  if (sbk == 1 && sbn % 8 == 0) return 2;
  return 0;
}

}  // namespace tsb

using namespace tsb;

extern "C" int tsb_gemm(const void *a, const void *b, void *c, int32_t dtype, int64_t M, int64_t N, int64_t K,
                        int64_t stride_am, int64_t stride_ak, int64_t stride_bk, int64_t stride_bn,
                        int64_t stride_cm, int64_t stride_cn, int32_t block_m, int32_t block_n,
                        int32_t block_k, const int32_t *tile_of_pid, int64_t n_programs, int64_t pid_lo,
                        int64_t pid_hi, int32_t *status, void *stream) {
  if (!a || !b || !c || !tile_of_pid) return fail(TSB_ERR_INVALID, "tsb_gemm: null pointer");
  if (M < 0 || N < 0 || K < 0 || block_m <= 0 || block_n <= 0 || block_k <= 0)
    return fail(TSB_ERR_INVALID, "tsb_gemm: negative size");
  if (pid_lo < 0 || pid_hi > n_programs || pid_lo > pid_hi)
    return fail(TSB_ERR_INVALID, "tsb_gemm: program range [%lld,%lld) outside %lld programs",
                (long long)pid_lo, (long long)pid_hi, (long long)n_programs);
  if (dtype != TSB_BF16 && dtype != TSB_F16 && dtype != TSB_F32)
    return fail(TSB_ERR_UNSUPPORTED, "tsb_gemm: dtype %d (f16, bf16 or f32)", dtype);
  if (pid_hi == pid_lo || M == 0 || N == 0) return TSB_OK;
  cudaStream_t s = (cudaStream_t)stream;

  const int mode = tensor_path_mode(a, b, dtype, stride_am, stride_ak, stride_bk, stride_bn, stride_cn, block_m,
                                    block_n, block_k);
  if (mode != 0) {
    const int is_bf16 = dtype == TSB_BF16;
    const int b_mn = mode == 1 ? 1 : 0;
    CUtensorMap map_a, map_b;
    // K == 0 needs no loads; give the encoder a non-empty extent
    const long long Kd = K > 0 ? K : 1;
    int rc = make_map(&map_a, a, is_bf16, Kd, M, stride_am, GEMM_BK, GEMM_BM);
    if (rc != TSB_OK) return rc;
    rc = b_mn ? make_map(&map_b, b, is_bf16, N, Kd, stride_bk, 64, GEMM_BK)
              : make_map(&map_b, b, is_bf16, Kd, N, stride_bn, GEMM_BK, block_n);
    if (rc != TSB_OK) return rc;
    GemmParams P;
    memset(&P, 0, sizeof(P));
    P.c = c;
    P.M = M; P.N = N; P.K = K;
    P.scm = stride_cm;
    P.tile_of_pid = tile_of_pid;
    P.pid_lo = pid_lo; P.pid_hi = pid_hi;
    P.status = status;
    P.block_n = block_n;
    P.k_sub = block_k / GEMM_BK;
    P.is_bf16 = is_bf16;
    P.b_mn_major = b_mn;
    P.c_vec_ok = ((uintptr_t)c % 16) == 0 && stride_cm % 8 == 0 && block_n % 8 == 0;
    int cols = 32;
    while (cols < 2 * block_n) cols *= 2;
    P.tmem_cols = cols;
    P.idesc = make_idesc(is_bf16, b_mn, GEMM_BM, block_n);
    const int stage_bytes = A_STAGE_BYTES + GEMM_BK * block_n * 2;
    int stages = (227 * 1024 - 2048) / stage_bytes;
    if (stages > 8) stages = 8;
    if (stages < 2) return fail(TSB_ERR_UNSUPPORTED, "tsb_gemm: block does not fit two pipeline stages");
    P.stages = stages;
    const int smem = stages * stage_bytes + 1024;
    static SmemLimit smem_limit;
    TSB_CUDA_OK(allow_dynamic_smem(gemm_tcgen05_kernel, smem, smem_limit));
    long long ctas = pid_hi - pid_lo;
    if (ctas > sm_count()) ctas = sm_count();
    gemm_tcgen05_kernel<<<(unsigned)ctas, GEMM_THREADS, smem, s>>>(map_a, map_b, P);
    TSB_LAUNCH_OK("gemm_tcgen05_kernel");
    return TSB_OK;
  }

  SimtParams Q;
  memset(&Q, 0, sizeof(Q));
  Q.a = a; Q.b = b; Q.c = c;
  Q.M = M; Q.N = N; Q.K = K;
  Q.sam = stride_am; Q.sak = stride_ak; Q.sbk = stride_bk; Q.sbn = stride_bn; Q.scm = stride_cm; Q.scn = stride_cn;
  Q.tile_of_pid = tile_of_pid;
  Q.pid_lo = pid_lo; Q.pid_hi = pid_hi;
  Q.block_m = block_m; Q.block_n = block_n;
  const long long progs = pid_hi - pid_lo;
  if (progs > 0x7fffffffll) return fail(TSB_ERR_UNSUPPORTED, "tsb_gemm: too many programs");
  dim3 grid((unsigned)progs, (unsigned)(((block_m + 63) / 64) * ((block_n + 63) / 64)));
  if (dtype == TSB_BF16) gemm_simt_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(Q);
  else if (dtype == TSB_F16) gemm_simt_kernel<__half><<<grid, 256, 0, s>>>(Q);
  else gemm_simt_kernel<float><<<grid, 256, 0, s>>>(Q);
  TSB_LAUNCH_OK("gemm_simt_kernel");
  return TSB_OK;
}

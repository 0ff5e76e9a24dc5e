// tt.dot path, two-CTA form: a pair of CTAs (a 2-CTA cluster on two SMs) computes two
// vertically adjacent 128 x BLOCK_N tiles of C with one tcgen05.mma.cta_group::2 stream.
//
// Same reference semantics as tsb_gemm.cu (MatmulConverter, ConversionPatterns.hpp:1128-1201;
// kernel-03-matrix-multiplication.mlir:157-204).  Why a second kernel: with one CTA per tile,
// every k-step moves A (16 KB) and the whole B block (32 KB) through that SM's shared memory,
// which holds the tensor pipe at ~69 % busy.  In the paired form each CTA stages its own A rows
// and only HALF of the B block; the MMA instruction (M = 256, issued by the even CTA) reads the
// A rows and the B half of both CTAs at the same shared-memory offsets and writes each CTA's
// 128 accumulator rows into that CTA's tensor memory.  Shared-memory traffic per SM drops by a
// third and six stages fit instead of four.
//
// Roles per CTA (192 threads): warp 0 lane 0 issues TMA loads (its own A tile and its B half;
// completion bytes are counted on the EVEN CTA's mbarrier), warp 1 lane 0 of the even CTA
// issues the MMAs and commits (multicast to both CTAs' barriers), warps 2-5 drain their own
// CTA's accumulator rows.  Loads are plain tile loads, no multicast.  Every wait is bounded in
// time; on expiry the CTA records where it stopped, both CTAs leave their loops, meet at the
// final cluster barrier, free tensor memory and return.
#include "tsb_tcgen05.cuh"
#include <string.h>

namespace tsb {

// ---- cta_group::2 and cluster PTX -------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local` (a shared::cta address) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// tile load whose completion bytes are counted on `bar` (a shared::cluster address, here the even CTA's)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives on the barrier at this offset in both CTAs once the MMAs issued so far have completed
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile(
      "{\n\t.reg .b16 m;\n\tmov.b16 m, 3;\n\t"
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n\t}"
      ::"r"(bar)
      : "memory");
}

constexpr int GEMM2_THREADS = 192;

struct Gemm2Params {
  void *c;
  long long M, N, K;
  long long scm;
  const int *pairs;     // (tile_m of the even CTA, tile_n) per pair of tiles
  long long n_pairs;
  int *status;
  int block_n;          // multiple of 32 (K-major B) or of 128 (MN-major B), <= 256
  int stages;
  int is_bf16;
  int b_mn_major;
  int c_vec_ok;
  int tmem_cols;
  uint32_t idesc;       // M = 256, N = block_n
};

__device__ __forceinline__ void give_up2(const Gemm2Params &P, volatile int *abort_flag, int role, long long item, int k) {
  if (atomicCAS((int *)abort_flag, 0, 1) == 0 && P.status) {
    P.status[1] = role + 10 * (int)cluster_ctarank();
    P.status[2] = (int)item;
    P.status[3] = k;
    __threadfence();
    atomicExch(&P.status[0], TSB_ERR_TIMEOUT);
  }
}

__global__ void __launch_bounds__(GEMM2_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const __grid_constant__ Gemm2Params P) {
  extern __shared__ uint8_t smem_raw[];
  // identical layout in both CTAs: the barrier at a given offset exists in each of them
  __shared__ __align__(8) unsigned long long bars[2 * 8 + 4];  // full[8], empty[8], tmem_full[2], tmem_empty[2]
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0: even CTA (issues the MMAs), 1: its peer
  const int BN = P.block_n, HN = BN / 2;
  const int S = P.stages;
  const uint32_t b_half_bytes = (uint32_t)GEMM_BK * HN * 2;
  const uint32_t stage_bytes = A_STAGE_BYTES + b_half_bytes;  // per CTA
  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  auto full_bar = [&](int s) { return smem_u32(&bars[s]); };
  auto empty_bar = [&](int s) { return smem_u32(&bars[8 + s]); };
  auto tfull_bar = [&](int a) { return smem_u32(&bars[16 + a]); };
  auto tempty_bar = [&](int a) { return smem_u32(&bars[18 + a]); };

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < S; ++s) {
      mbar_init(full_bar(s), 1);   // used in the even CTA only: its producer arms it for both CTAs' bytes
      mbar_init(empty_bar(s), 1);  // one multicast commit per use
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8);  // used in the even CTA only: four epilogue warps of each CTA
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 1) {
    tmem_alloc2(smem_u32(&tmem_base_slot), (uint32_t)P.tmem_cols);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  const long long cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  const int k_iters = (int)((P.K + GEMM_BK - 1) / GEMM_BK);
  // a CTA that gives up also raises its peer's flag so that both leave their loops promptly
  auto raise_peer = [&]() {
    const uint32_t remote = map_to_cta(smem_u32(&abort_flag), rank ^ 1u);
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(remote), "r"(1) : "memory");
  };

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      int s = 0;
      uint32_t phase = 0;
      long long issued = 0;
      bool ok = true;
      for (long long w = cluster_id; w < P.n_pairs && ok; w += n_clusters) {
        const int tm = P.pairs[2 * w] + (int)rank, tn = P.pairs[2 * w + 1];
        for (int k = 0; k < k_iters; ++k) {
          if (!mbar_wait(empty_bar(s), phase ^ 1u, &abort_flag)) {
            give_up2(P, &abort_flag, 0, w, k);
            raise_peer();
            ok = false;
            break;
          }
          const uint32_t a_dst = smem0 + (uint32_t)s * stage_bytes;
          const uint32_t b_dst = a_dst + A_STAGE_BYTES;
          if (rank == 0) mbar_expect_tx(full_bar(s), 2u * stage_bytes);
          const uint32_t bar = map_to_cta(full_bar(s), 0);  // bytes are counted in the even CTA
          tma_load_2d_pair(a_dst, &map_a, k * GEMM_BK, tm * GEMM_BM, bar);
          const int n0 = tn * BN + (int)rank * HN;  // this CTA's half of the B block
          if (P.b_mn_major) {
            for (int c = 0; c < HN / 64; ++c)
              tma_load_2d_pair(b_dst + (uint32_t)c * (GEMM_BK * 128), &map_b, n0 + c * 64, k * GEMM_BK, bar);
          } else {
            tma_load_2d_pair(b_dst, &map_b, k * GEMM_BK, n0, bar);
          }
          ++issued;
          if (++s == S) { s = 0; phase ^= 1u; }
        }
      }
      if (!ok || abort_flag) {
        // drain: the even CTA's full barriers cover both CTAs' copies; the peer waits the same
        // bounded time on its own (never completing) copy so that its loads have landed
        const long long pending = issued < S ? issued : S;
        int ds = s;
        uint32_t dphase = phase;
        for (long long i = 0; i < pending; ++i) {
          if (--ds < 0) { ds = S - 1; dphase ^= 1u; }
          if (rank == 0) mbar_wait(full_bar(ds), dphase, &abort_flag, DRAIN_LIMIT_NS);
        }
        if (rank != 0) {
          const unsigned long long t0 = global_ns();
          while (global_ns() - t0 < DRAIN_LIMIT_NS) {}
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (even CTA only) ----------------
    if (lane == 0 && rank == 0) {
      int s = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (long long w = cluster_id; w < P.n_pairs && ok; w += n_clusters) {
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, &abort_flag)) {
          give_up2(P, &abort_flag, 1, w, -1);
          raise_peer();
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int k = 0; k < k_iters; ++k) {
          if (!mbar_wait(full_bar(s), phase, &abort_flag)) {
            give_up2(P, &abort_flag, 1, w, k);
            raise_peer();
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_src = smem0 + (uint32_t)s * stage_bytes;
          const uint32_t b_src = a_src + A_STAGE_BYTES;
#pragma unroll
          for (int kk = 0; kk < GEMM_BK / 16; ++kk) {
            const uint64_t ad = make_smem_desc(a_src + kk * 32, 16, 1024);
            const uint64_t bd = P.b_mn_major ? make_smem_desc(b_src + kk * 16 * 128, GEMM_BK * 128, 1024)
                                             : make_smem_desc(b_src + kk * 32, 16, 1024);
            umma_f16_pair(d_tmem, ad, bd, P.idesc, (k > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit_pair(empty_bar(s));  // frees this stage in both CTAs
          if (++s == S) { s = 0; phase ^= 1u; }
        }
        if (ok) umma_commit_pair(tfull_bar(acc));  // accumulators of both CTAs are complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ---------------- epilogue (both CTAs, own accumulator rows) ----------------
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (long long w = cluster_id; w < P.n_pairs; w += n_clusters) {
      const int tm = P.pairs[2 * w] + (int)rank, tn = P.pairs[2 * w + 1];
      if (!mbar_wait(tfull_bar(acc), acc_phase, &abort_flag)) {
        give_up2(P, &abort_flag, 2, w, -1);
        if (lane == 0) raise_peer();
        break;
      }
      tc_fence_after();
      const long long row = (long long)tm * GEMM_BM + q * 32 + lane;
      const long long col0 = (long long)tn * BN;
      for (int c = 0; c < BN; c += 32) {
        uint32_t v[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c), v);
        tmem_ld_wait();
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
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while its peer may still touch its memory or barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, (uint32_t)P.tmem_cols);
  }
}

}  // namespace tsb

using namespace tsb;

extern "C" int tsb_gemm_paired(const void *a, const void *b, void *c, int32_t dtype, int64_t M, int64_t N,
                               int64_t K, int64_t stride_am, int64_t stride_ak, int64_t stride_bk,
                               int64_t stride_bn, int64_t stride_cm, int64_t stride_cn, int32_t block_m,
                               int32_t block_n, int32_t block_k, const int32_t *pairs, int64_t n_pairs,
                               int32_t *status, void *stream) {
  if (!a || !b || !c || !pairs) return fail(TSB_ERR_INVALID, "tsb_gemm_paired: null pointer");
  if (M < 0 || N < 0 || K < 0 || n_pairs < 0) return fail(TSB_ERR_INVALID, "tsb_gemm_paired: negative size");
  if (n_pairs == 0 || M == 0 || N == 0) return TSB_OK;
  const int mode = tensor_path_mode(a, b, dtype, stride_am, stride_ak, stride_bk, stride_bn, stride_cn, block_m,
                                    block_n, block_k);
  if (mode == 0 || K == 0)
    return fail(TSB_ERR_UNSUPPORTED, "tsb_gemm_paired: operands are not eligible for the tensor-core path");
  const int half_n = block_n / 2;
  if ((mode == 1 && half_n % 64 != 0) || (mode == 2 && half_n % 16 != 0))
    return fail(TSB_ERR_UNSUPPORTED, "tsb_gemm_paired: BLOCK_N = %d cannot be split between two CTAs", block_n);
  const int is_bf16 = dtype == TSB_BF16;
  const int b_mn = mode == 1 ? 1 : 0;
  CUtensorMap map_a, map_b;
  int rc = make_map(&map_a, a, is_bf16, K, M, stride_am, GEMM_BK, GEMM_BM);
  if (rc != TSB_OK) return rc;
  rc = b_mn ? make_map(&map_b, b, is_bf16, N, K, stride_bk, 64, GEMM_BK)
            : make_map(&map_b, b, is_bf16, K, N, stride_bn, GEMM_BK, half_n);
  if (rc != TSB_OK) return rc;
  Gemm2Params P;
  memset(&P, 0, sizeof(P));
  P.c = c;
  P.M = M; P.N = N; P.K = K;
  P.scm = stride_cm;
  P.pairs = pairs;
  P.n_pairs = n_pairs;
  P.status = status;
  P.block_n = block_n;
  P.is_bf16 = is_bf16;
  P.b_mn_major = b_mn;
  P.c_vec_ok = ((uintptr_t)c % 16) == 0 && stride_cm % 8 == 0 && block_n % 8 == 0;
  int cols = 32;
  while (cols < 2 * block_n) cols *= 2;
  P.tmem_cols = cols;
  P.idesc = make_idesc(is_bf16, b_mn, 2 * GEMM_BM, block_n);
  const int stage_bytes = A_STAGE_BYTES + GEMM_BK * half_n * 2;
  int stages = (220 * 1024) / stage_bytes;
  if (stages > 8) stages = 8;
  if (stages < 2) return fail(TSB_ERR_UNSUPPORTED, "tsb_gemm_paired: block does not fit two pipeline stages");
  P.stages = stages;
  const int smem = stages * stage_bytes + 1024;
  static SmemLimit smem_limit;
  TSB_CUDA_OK(allow_dynamic_smem(gemm_tcgen05_pair_kernel, smem, smem_limit));
  long long clusters = n_pairs;
  const long long max_clusters = sm_count() / 2;
  if (clusters > max_clusters) clusters = max_clusters;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)(2 * clusters), 1, 1);
  cfg.blockDim = dim3(GEMM2_THREADS, 1, 1);
  cfg.dynamicSmemBytes = (size_t)smem;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  TSB_CUDA_OK(cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_kernel, map_a, map_b, P));
  return TSB_OK;
}

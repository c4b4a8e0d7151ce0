// bf16 GEMM for sm_100a: D[M,N] = op(A) * op(B), fp32 accumulation in tensor memory.
//
// Replaces the cuBLAS calls behind every F.linear / matmul of the reference model
// (picotron/model.py:124-126,161,186,212; backward dX = dY*W and dW = dY^T*X).
//
// Structure (one persistent CTA per SM, 192 threads, no clusters, no TMA multicast):
//   warp 0      TMA producer: fills a 4-stage shared-memory ring with 128xBK A tiles and 256xBK B tiles
//               (128-byte swizzle), one mbarrier (expect_tx) per stage.
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=256, K=16) from shared-memory
//               descriptors into one of two 256-column TMEM accumulators; tcgen05.commit releases the
//               shared-memory stage and, after the last k-block, publishes the accumulator.
//   warps 2-5   epilogue: tcgen05.ld the accumulator (each warp owns 32 TMEM lanes = 32 rows), convert
//               and store bf16, or read-modify-write an fp32 destination (D += acc) -- this is how weight
//               gradients are accumulated straight into the fp32 gradient buckets. The epilogue of tile
//               i overlaps the main loop of tile i+1 through the double-buffered accumulator.
//
// Operand layouts. "K-major" means the reduction dimension is contiguous in memory, "MN-major" means the
// M (or N) dimension is contiguous. All three combinations the model needs are served by the same kernel:
//   forward  Y = X W^T : A = X [M,K] K-major,  B = W [N,K] K-major
//   dgrad   dX = dY W  : A = dY [M,K] K-major, B = W [K,N] MN-major
//   wgrad   dW = dY^T X: A = dY [K,M] MN-major, B = X [K,N] MN-major
// MN-major tiles are loaded as 64-element-wide column chunks (one TMA box of 64 x BK each) so that every
// chunk is a canonical 128-byte-swizzled UMMA block; the descriptor's leading-dimension offset walks
// the chunks and its stride offset walks groups of eight k rows.
#include <stdlib.h>
#include "common.cuh"
#include "tensormap.cuh"

// process-wide count of kernel launches issued by this library (read by the benchmark)
static unsigned long long g_launch_count = 0;
extern "C" void pt_count_launches(int n) { g_launch_count += (unsigned long long)n; }
extern "C" unsigned long long pt_launch_count() { return g_launch_count; }

namespace pt {
namespace gemm {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_BYTES = BN * BK * 2;  // 32 KiB
constexpr int SMEM_BYTES = STAGES * (A_BYTES + B_BYTES) + 1024;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr unsigned KERNEL_ID = 1;

enum OutMode { OUT_BF16 = 0, OUT_F32_ACC = 1, OUT_F32 = 2 };

struct Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int& m_blk, int& n_blk) {
  constexpr int GROUP_M = 8;
  const int per_group = GROUP_M * num_n;
  const int group = t / per_group;
  const int first_m = group * GROUP_M;
  const int gsize = min(num_m - first_m, GROUP_M);
  const int r = t - group * per_group;
  m_blk = first_m + r % gsize;
  n_blk = r / gsize;
}

template <bool A_MN, bool B_MN, int OUT_MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 void* __restrict__ Dptr, int M, int N, int K, long long ldd, KernelStatus* status) {
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  __shared__ Barriers bars;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + STAGES * A_BYTES;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (M + BM - 1) / BM;
  const int num_n = (N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars.full[s], 1);
      mbar_init(&bars.empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars.tmem_full[s], 1);
      mbar_init(&bars.tmem_empty[s], 4);
    }
    bars.abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(&bars.tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  pdl_wait();                      // the prologue above ran under the predecessor's tail; its results are needed from here on
  const uint32_t tmem_base = bars.tmem_base;
  volatile int* abort_flag = &bars.abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int m_blk, n_blk;
        tile_coords(t, num_m, num_n, m_blk, n_blk);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&bars.empty[stage], phase ^ 1, abort_flag)) {
            report_error(status, KERNEL_ID, 1);
            ok = false;
            break;
          }
          mbar_expect_tx(&bars.full[stage], A_BYTES + B_BYTES);
          uint8_t* sa = smem_a + stage * A_BYTES;
          uint8_t* sb = smem_b + stage * B_BYTES;
          if (!A_MN) {
            tma_load_2d(sa, &tma_a, &bars.full[stage], kb * BK, m_blk * BM);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_2d(sa + c * (BK * 128), &tma_a, &bars.full[stage], m_blk * BM + c * 64, kb * BK);
          }
          if (!B_MN) {
            tma_load_2d(sb, &tma_b, &bars.full[stage], kb * BK, n_blk * BN);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sb + c * (BK * 128), &tma_b, &bars.full[stage], n_blk * BN + c * 64, kb * BK);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int local = 0;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&bars.tmem_empty[acc], acc_phase ^ 1, abort_flag)) {
          report_error(status, KERNEL_ID, 2);
          ok = false;
          break;
        }
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&bars.full[stage], phase, abort_flag)) {
            report_error(status, KERNEL_ID, 3);
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const uint32_t sa = smem_u32(smem_a + stage * A_BYTES);
          const uint32_t sb = smem_u32(smem_b + stage * B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t a_desc = A_MN ? make_smem_desc_sw128(sa + k * (UMMA_K * 128), BK * 128, 1024)
                                         : make_smem_desc_sw128(sa + k * (UMMA_K * 2), 16, 1024);
            const uint64_t b_desc = B_MN ? make_smem_desc_sw128(sb + k * (UMMA_K * 128), BK * 128, 1024)
                                         : make_smem_desc_sw128(sb + k * (UMMA_K * 2), 16, 1024);
            umma_bf16(d_tmem, a_desc, b_desc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&bars.empty[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&bars.tmem_full[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) are accessible to this warp
    bool ok = true;
    int local = 0;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++local) {
      int m_blk, n_blk;
      tile_coords(t, num_m, num_n, m_blk, n_blk);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      if (!mbar_wait(&bars.tmem_full[acc], acc_phase, abort_flag)) {
        if (lane == 0) report_error(status, KERNEL_ID, 4);
        ok = false;
        break;
      }
      tcgen05_fence_after();
      const int row = m_blk * BM + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN;
      // Software-pipelined drain of the accumulator: the TMEM load of chunk c+1 is in flight while chunk c is stored.
      auto store_chunk = [&](const uint32_t (&r)[32], int c) {
        const int col0 = n_blk * BN + c * 32;
        if (row < M && col0 < N) {
          if (OUT_MODE == OUT_BF16) {
            __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(Dptr) + (long long)row * ldd + col0;
            if (col0 + 32 <= N) {
              uint4* d4 = reinterpret_cast<uint4*>(drow);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4 v;
                v.x = pack_bf16(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
                v.y = pack_bf16(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
                v.z = pack_bf16(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
                v.w = pack_bf16(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
                d4[j] = v;
              }
            } else {
              for (int j = 0; j < 32 && col0 + j < N; ++j) drow[j] = __float2bfloat16(__uint_as_float(r[j]));
            }
          } else {
            float* drow = reinterpret_cast<float*>(Dptr) + (long long)row * ldd + col0;
            if (col0 + 32 <= N) {
              float4* d4 = reinterpret_cast<float4*>(drow);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float4 v = make_float4(__uint_as_float(r[4 * j + 0]), __uint_as_float(r[4 * j + 1]),
                                       __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                if (OUT_MODE == OUT_F32_ACC) {
                  const float4 o = d4[j];
                  v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                }
                d4[j] = v;
              }
            } else {
              for (int j = 0; j < 32 && col0 + j < N; ++j) {
                float v = __uint_as_float(r[j]);
                if (OUT_MODE == OUT_F32_ACC) v += drow[j];
                drow[j] = v;
              }
            }
          }
        }
            };
      {
        uint32_t ra[32], rb[32];
        tmem_ld_32x32b_x32(t_row, ra);
#pragma unroll
        for (int c = 0; c < BN / 32; c += 2) {
          tmem_ld_wait();
          tmem_ld_32x32b_x32(t_row + (c + 1) * 32, rb);
          store_chunk(ra, c);
          tmem_ld_wait();
          if (c + 2 < BN / 32) tmem_ld_32x32b_x32(t_row + (c + 2) * 32, ra);
          store_chunk(rb, c + 1);
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars.tmem_empty[acc]);
    }
  }

  // ------------------------------------------------------------------ teardown
  tcgen05_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // give copies that are still in flight time to land before shared memory is released
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
static int make_map_2d(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                       uint32_t box_inner, uint32_t box_outer) {
  return make_bf16_map_2d(map, base, inner, outer, ld, box_inner, box_outer);
}

static KernelStatus* g_status[64] = {nullptr};

KernelStatus* status_word() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  if (g_status[dev] == nullptr) {
    KernelStatus* p = nullptr;
    if (cudaMalloc(&p, sizeof(KernelStatus)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, sizeof(KernelStatus));
    g_status[dev] = p;
  }
  return g_status[dev];
}

template <bool A_MN, bool B_MN, int OUT_MODE>
static int launch(const CUtensorMap& ma, const CUtensorMap& mb, void* D, int M, int N, int K, long long ldd,
                  int num_sms, cudaStream_t stream) {
  auto kern = gemm_bf16_kernel<A_MN, B_MN, OUT_MODE>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -3;
    configured = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  const cudaError_t err = launch_pdl(kern, dim3(grid), dim3(NUM_THREADS), SMEM_BYTES, stream, ma, mb, D, M, N, K, ldd, status_word());
  pt_count_launches(1);
  return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? 0 : -4;
}

}  // namespace gemm
}  // namespace pt

// D[M,N] = op(A) op(B).
//   a_mn == 0: A is [M,K] row-major (row stride lda);  a_mn == 1: A is stored [K,M] row-major.
//   b_mn == 0: B is [N,K] row-major (row stride ldb);  b_mn == 1: B is stored [K,N] row-major.
//   out_mode 0: D bf16 = acc;  1: D fp32 += acc;  2: D fp32 = acc.   ldd = row stride of D in elements.
// Requirements: 16-byte aligned bases, lda/ldb multiples of 8, ldd multiple of 8 (bf16) or 4 (fp32).
// Returns 0 on success, negative on a host-side error.
extern "C" int pt_gemm_bf16_pair(const void* A, const void* B, void* D, int M, int N, int K, long long lda,
                                 long long ldb, long long ldd, int a_mn, int b_mn, int out_mode, void* status,
                                 cudaStream_t stream);

// 1: 256x256 tiles on CTA pairs (default), 0: 128x256 tiles on single CTAs.
static int g_use_pair = 1;
extern "C" void pt_gemm_set_pair(int on) { g_use_pair = on; }
extern "C" int pt_gemm_get_pair() { return g_use_pair; }

extern "C" int pt_gemm_bf16(const void* A, const void* B, void* D, int M, int N, int K, long long lda, long long ldb,
                            long long ldd, int a_mn, int b_mn, int out_mode, int num_sms, cudaStream_t stream) {
  using namespace pt::gemm;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (reinterpret_cast<uintptr_t>(D) & 15) || (out_mode == OUT_BF16 ? (ldd % 8) : (ldd % 4)))
    return -10;
  if (g_use_pair) {
    const int rc = pt_gemm_bf16_pair(A, B, D, M, N, K, lda, ldb, ldd, a_mn, b_mn, out_mode, status_word(), stream);
    if (rc != -5) return rc;
    g_use_pair = 0;  // CTA pairs cannot be scheduled on this device/partition: use single-CTA tiles from now on
  }
  CUtensorMap ma, mb;
  int rc;
  rc = a_mn ? make_map_2d(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 64, BK)
            : make_map_2d(&ma, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, BM);
  if (rc) return rc;
  rc = b_mn ? make_map_2d(&mb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, BK)
            : make_map_2d(&mb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, BN);
  if (rc) return rc;
#define PT_GEMM_CASE(AM, BMN, OM) \
  if (a_mn == AM && b_mn == BMN && out_mode == OM) return launch<AM, BMN, OM>(ma, mb, D, M, N, K, ldd, num_sms, stream);
  PT_GEMM_CASE(0, 0, 0) PT_GEMM_CASE(0, 0, 1) PT_GEMM_CASE(0, 0, 2)
  PT_GEMM_CASE(0, 1, 0) PT_GEMM_CASE(0, 1, 1) PT_GEMM_CASE(0, 1, 2)
  PT_GEMM_CASE(1, 1, 0) PT_GEMM_CASE(1, 1, 1) PT_GEMM_CASE(1, 1, 2)
  PT_GEMM_CASE(1, 0, 0) PT_GEMM_CASE(1, 0, 1) PT_GEMM_CASE(1, 0, 2)
#undef PT_GEMM_CASE
  return -11;
}

extern "C" void* pt_status_word() { return pt::gemm::status_word(); }

// Programmatic dependent launch of the step's kernels (common.cuh): on unless PICOTRON_PDL=0 or pt_set_pdl(0).
static int g_pdl = -1;
extern "C" int pt_pdl_enabled() {
  if (g_pdl < 0) {
    const char* e = getenv("PICOTRON_PDL");
    g_pdl = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return g_pdl;
}
extern "C" void pt_set_pdl(int on) { g_pdl = on ? 1 : 0; }

// Reads and clears the per-device kernel status word. 0 = no kernel reported a timed-out wait.
extern "C" unsigned int pt_kernel_status_fetch_and_clear() {
  pt::KernelStatus* p = pt::gemm::status_word();
  if (p == nullptr) return 0;
  pt::KernelStatus h;
  if (cudaMemcpy(&h, p, sizeof(h), cudaMemcpyDeviceToHost) != cudaSuccess) return 0xffffffffu;
  if (h.code != 0) cudaMemset(p, 0, sizeof(h));
  return h.code;
}

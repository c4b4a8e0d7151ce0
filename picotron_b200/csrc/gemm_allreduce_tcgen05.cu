// Tensor-parallel GEMM fused with its all-reduce (sm_100a, CTA pairs): D = sum over ranks of op(A_r) * op(B_r).
//
// Replaces "F.linear, then dist.all_reduce" of the reference's RowParallelLinear forward
// (picotron/tensor_parallel/tensor_parallel.py:184-189) and "grad_input GEMM, then all_reduce" of the
// column-parallel backward (picotron/tensor_parallel/tp_communications.py:29-33,92-100) by ONE kernel in which the
// reduction of finished output tiles over NVLink overlaps the MMAs of the following tiles.
//
// It is the CTA-pair GEMM of gemm_pair_tcgen05.cu (same operand layouts, same TMA/MMA roles, bf16 output written by
// the epilogue threads themselves because the reducer must see complete half tiles) plus a fourth role. It is used where
// the reduction goes through the NVSwitch (groups of 4+ ranks); between 2 ranks the plain GEMM followed by the push
// all-reduce of csrc/comm.cu is faster and is what the tensor-parallel layers run. D lives in a symmetric buffer (same offset at every rank). Output tiles are owned round-robin by the ranks;
// all ranks walk the tiles in the same order with the same grid (the launcher fixes the grid from the shape alone).
//   epilogue   writes the bf16 partial half-tile (128 rows x 256 columns per CTA) into the LOCAL buffer, then stores
//              "rank r finished half-tile h of tile t" into the flag array of the tile's OWNER rank (release, system scope).
//   reducer    (4 extra warps per CTA) on the owner: waits -- bounded -- until every rank's flag for its half-tile shows
//              this call's epoch, loads the half-tile from every rank (plain peer loads), sums in fp32, stores the bf16
//              result into every rank's buffer (plain peer stores) and sets the tile's "done" flag at every rank.
//   kernel end every CTA waits -- bounded -- for the done flags of the tiles it computed, so when the kernel finishes the
//              local buffer holds the fully reduced D.
// Only reducers wait on other ranks, and they wait for work that no rank makes conditional on a reducer, so the
// cross-rank dependency graph is acyclic. No TMA load uses multicast; remote data moves with ordinary loads and stores.
#include "common.cuh"
#include "tensormap.cuh"

extern "C" void pt_count_launches(int n);

namespace pt {
namespace gemm_ar {

constexpr int BM = 128;        // rows of A per CTA (256 per pair)
constexpr int BN_HALF = 128;   // columns of B per CTA (256 per pair)
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK * 2;        // 16 KiB
constexpr int B_BYTES = BN_HALF * BK * 2;   // 16 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;
constexpr int NUM_THREADS = 320;      // producer, MMA, 4 epilogue warps, 4 reducer warps
constexpr int TMEM_COLS = 512;
constexpr unsigned KERNEL_ID = 6;
constexpr int MAX_RANKS = 8;
constexpr int MAX_TILES = 1024;
// layout of the per-rank flag region used by this kernel (uint32 words), after the 16 KiB of barrier flags
constexpr size_t FLAG_WORDS_OFFSET = 16384 / 4;
constexpr size_t START_WORDS = (size_t)MAX_TILES * 2 * MAX_RANKS;   // [tile][half][source rank]
// call counter of the workspace: two control words behind the 8 KiB of barrier flags (shared with csrc/comm.cu, which
// documents the protocol: every CTA reads counter + 1 as this launch's epoch, the last CTA to finish stores it back)
constexpr size_t CTRL_WORDS_OFFSET = 8192 / 4;

struct Peers {
  void* buf[MAX_RANKS];            // data region base of every rank (peer mapped)
  unsigned int* flags[MAX_RANKS];  // flag region base of every rank
};

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool wait_flag(const unsigned int* p, unsigned int epoch, unsigned long long wait_ns) {
  const unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  while ((int)(ld_acquire_sys(p) - epoch) < 0) {
    if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > wait_ns) return false;
  }
  return true;
}
__device__ __forceinline__ void named_barrier(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

struct Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int& m_blk, int& n_blk) {
  constexpr int GROUP_M = 4;   // 4 x 256 rows
  const int per_group = GROUP_M * num_n;
  const int group = t / per_group;
  const int first_m = group * GROUP_M;
  const int gsize = min(num_m - first_m, GROUP_M);
  const int r = t - group * per_group;
  m_blk = first_m + r % gsize;
  n_blk = r / gsize;
}

// Rank that reduces tile t. Consecutive tiles of one cluster (t, t + num_clusters, ...) rotate over the ranks so that every
// CTA pair reduces only every world-th tile it computes, whatever the parity of num_clusters.
__device__ __forceinline__ int tile_owner(int t, int num_clusters, int world) {
  return (t / num_clusters + t % num_clusters) % world;
}

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_ar_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, Peers peers,
               __nv_bfloat16* mc_base, long long d_offset, int M, int N, int K, long long ldd, int my_rank, int world,
               unsigned long long wait_ns, KernelStatus* status) {
  unsigned int* ctrl = peers.flags[my_rank] + CTRL_WORDS_OFFSET;
  const unsigned int epoch = *reinterpret_cast<volatile unsigned int*>(ctrl) + 1u;
  void* __restrict__ Dptr = reinterpret_cast<__nv_bfloat16*>(peers.buf[my_rank]) + d_offset;
  extern __shared__ uint8_t smem_raw[];
  __shared__ Barriers bars;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + STAGES * A_BYTES;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();           // 0 = leader
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;
  const int num_m = (M + 2 * BM - 1) / (2 * BM);
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
      mbar_init(&bars.tmem_empty[s], 8);    // 4 epilogue warps x 2 CTAs (used in the leader only)
    }
    bars.abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(&bars.tmem_base, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  tcgen05_fence_after();
  const uint32_t tmem_base = bars.tmem_base;
  volatile int* abort_flag = &bars.abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
        int m_blk, n_blk;
        tile_coords(t, num_m, num_n, m_blk, n_blk);
        const int row0 = m_blk * 2 * BM + (int)rank * BM;          // this CTA's rows of A
        const int col0 = n_blk * BN + (int)rank * BN_HALF;         // this CTA's columns of B
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&bars.empty[stage], phase ^ 1, abort_flag)) {
            report_error(status, KERNEL_ID, 1);
            ok = false;
            break;
          }
          const uint32_t full_leader = mapa_u32(smem_u32(&bars.full[stage]), 0);
          if (rank == 0) mbar_expect_tx(&bars.full[stage], 2 * STAGE_BYTES);
          uint8_t* sa = smem_a + stage * A_BYTES;
          uint8_t* sb = smem_b + stage * B_BYTES;
          if (!A_MN) {
            tma_load_2d_pair(sa, &tma_a, full_leader, kb * BK, row0);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_2d_pair(sa + c * (BK * 128), &tma_a, full_leader, row0 + c * 64, kb * BK);
          }
          if (!B_MN) {
            tma_load_2d_pair(sb, &tma_b, full_leader, kb * BK, col0);
          } else {
#pragma unroll
            for (int c = 0; c < BN_HALF / 64; ++c)
              tma_load_2d_pair(sb + c * (BK * 128), &tma_b, full_leader, col0 + c * 64, kb * BK);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int local = 0;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++local) {
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
            umma_bf16_pair(d_tmem, a_desc, b_desc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          const uint32_t e = smem_u32(&bars.empty[stage]);
          umma_commit_pair(mapa_u32(e, 0));
          umma_commit_pair(mapa_u32(e, 1));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) {
          const uint32_t f = smem_u32(&bars.tmem_full[acc]);
          umma_commit_pair(mapa_u32(f, 0));
          umma_commit_pair(mapa_u32(f, 1));
        }
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int quarter = warp & 3;
    bool ok = true;
    int local = 0;
    for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++local) {
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
      const int row = m_blk * 2 * BM + (int)rank * BM + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN;
      // Software-pipelined drain of the accumulator: the TMEM load of chunk c+1 is in flight while chunk c is stored.
      auto store_chunk = [&](const uint32_t (&r)[32], int c) {
        const int col0 = n_blk * BN + c * 32;
        if (row < M && col0 < N) {
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
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&bars.tmem_empty[acc]), 0));
      // the whole half-tile is in the local buffer: tell the tile's owner
      named_barrier(1, 128);
      if (warp == 2 && lane == 0) {
        __threadfence_system();
        const int owner = tile_owner(t, num_clusters, world);
        st_release_sys(peers.flags[owner] + FLAG_WORDS_OFFSET + ((size_t)t * 2 + rank) * MAX_RANKS + my_rank, epoch);
      }
    }
  } else {
    // ------------------------------------------------------------------ reducer (warps 6..9 of both CTAs)
    const int rt = threadIdx.x - 192;            // 0..127
    bool ok = true;
    for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
      if (tile_owner(t, num_clusters, world) != my_rank) continue;
      int m_blk, n_blk;
      tile_coords(t, num_m, num_n, m_blk, n_blk);
      if (rt < world) {
        if (!wait_flag(peers.flags[my_rank] + FLAG_WORDS_OFFSET + ((size_t)t * 2 + rank) * MAX_RANKS + rt, epoch, wait_ns)) {
          report_error(status, KERNEL_ID, 5);
          *abort_flag = 1;
        }
      }
      named_barrier(2, 128);
      if (*abort_flag) { ok = false; break; }
      // half-tile: 128 rows x 256 columns = 128 x 32 units of 8 bf16; thread rt walks units rt, rt+128, ...
      const int row0 = m_blk * 2 * BM + (int)rank * BM;
      const int col0 = n_blk * BN;
      // Microsecond NVLink latency: keep many 16-byte transactions in flight per thread.
      if (mc_base != nullptr) {
        // NVSwitch path: one multimem.ld_reduce returns the sum over all ranks, one multimem.st writes it to all ranks
        constexpr int BATCH = 16;
#pragma unroll 1
        for (int u0 = rt; u0 < 128 * 32; u0 += 128 * BATCH) {
          uint4 v[BATCH];
#pragma unroll
          for (int j = 0; j < BATCH; ++j) {
            const int u = u0 + j * 128;
            const int r = row0 + (u >> 5), c = col0 + (u & 31) * 8;
            if (r < M && c < N) {
              __nv_bfloat16* a = mc_base + d_offset + (long long)r * ldd + c;
              asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                           : "=r"(v[j].x), "=r"(v[j].y), "=r"(v[j].z), "=r"(v[j].w) : "l"(a) : "memory");
            }
          }
#pragma unroll
          for (int j = 0; j < BATCH; ++j) {
            const int u = u0 + j * 128;
            const int r = row0 + (u >> 5), c = col0 + (u & 31) * 8;
            if (r < M && c < N) {
              __nv_bfloat16* a = mc_base + d_offset + (long long)r * ldd + c;
              asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(a), "r"(v[j].x),
                           "r"(v[j].y), "r"(v[j].z), "r"(v[j].w) : "memory");
            }
          }
        }
      } else {
        constexpr int BATCH = 8;
#pragma unroll 1
        for (int u0 = rt; u0 < 128 * 32; u0 += 128 * BATCH) {
          float acc8[BATCH][8];
#pragma unroll
          for (int j = 0; j < BATCH; ++j)
#pragma unroll
            for (int e = 0; e < 8; ++e) acc8[j][e] = 0.f;
          for (int q = 0; q < world; ++q) {
            uint4 v[BATCH];
#pragma unroll
            for (int j = 0; j < BATCH; ++j) {
              const int u = u0 + j * 128;
              const int r = row0 + (u >> 5), c = col0 + (u & 31) * 8;
              v[j] = make_uint4(0, 0, 0, 0);
              if (r < M && c < N)
                v[j] = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(peers.buf[q]) + d_offset +
                                                       (long long)r * ldd + c);
            }
#pragma unroll
            for (int j = 0; j < BATCH; ++j) {
              const uint32_t w4[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w4[e]));
                acc8[j][2 * e] += f.x;
                acc8[j][2 * e + 1] += f.y;
              }
            }
          }
#pragma unroll
          for (int j = 0; j < BATCH; ++j) {
            const int u = u0 + j * 128;
            const int r = row0 + (u >> 5), c = col0 + (u & 31) * 8;
            if (r < M && c < N) {
              const uint4 o = make_uint4(pack_bf16(acc8[j][0], acc8[j][1]), pack_bf16(acc8[j][2], acc8[j][3]),
                                         pack_bf16(acc8[j][4], acc8[j][5]), pack_bf16(acc8[j][6], acc8[j][7]));
              for (int q = 0; q < world; ++q)
                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(peers.buf[q]) + d_offset + (long long)r * ldd + c) = o;
            }
          }
        }
      }
      __threadfence_system();
      named_barrier(2, 128);
      if (rt < world)
        st_release_sys(peers.flags[rt] + FLAG_WORDS_OFFSET + START_WORDS + (size_t)t * 2 + rank, epoch);
    }
    // every tile this CTA computed must have been reduced (by its owner) before the kernel may end
    if (ok) {
      for (int t = cluster_id + rt * num_clusters; t < num_tiles; t += 128 * num_clusters) {
        if (!wait_flag(peers.flags[my_rank] + FLAG_WORDS_OFFSET + START_WORDS + (size_t)t * 2 + rank, epoch, wait_ns)) {
          report_error(status, KERNEL_ID, 6);
          *abort_flag = 1;
          break;
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tcgen05_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  cluster_arrive();
  cluster_wait();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0) {            // advance the workspace's call counter once every CTA of this launch is through
    __threadfence();
    const unsigned int arrived = atomicAdd(ctrl + 1, 1u);
    if (arrived == gridDim.x - 1) {
      ctrl[1] = 0u;
      __threadfence();
      *reinterpret_cast<volatile unsigned int*>(ctrl) = epoch;
    }
  }
}

template <bool A_MN, bool B_MN>
static int launch(const CUtensorMap& ma, const CUtensorMap& mb, const Peers& peers, void* mc_ptr, long long d_offset, int M, int N, int K,
                  long long ldd, int rank, int world, unsigned long long wait_ns, int clusters_cap, KernelStatus* status,
                  cudaStream_t stream) {
  auto kern = gemm_ar_kernel<A_MN, B_MN>;
  static int max_clusters = 0;
  if (max_clusters == 0) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -3;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2, 1, 1);
    cfg.blockDim = dim3(NUM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      return -5;
    }
    max_clusters = n;
  }
  const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
  if (tiles > MAX_TILES) return -12;
  if (clusters_cap <= 0) return max_clusters;     // query mode: how many CTA pairs fit on this device
  const int cap = clusters_cap < max_clusters ? clusters_cap : max_clusters;
  if (cap != clusters_cap) return -13;            // the agreed grid does not fit here: ranks would disagree on tile owners
  const int clusters = tiles < cap ? tiles : cap;
  kern<<<2 * clusters, NUM_THREADS, SMEM_BYTES, stream>>>(ma, mb, peers, (__nv_bfloat16*)mc_ptr, d_offset, M, N, K, ldd, rank, world, wait_ns, status);
  pt_count_launches(1);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace gemm_ar
}  // namespace pt

extern "C" void* pt_status_word();
extern "C" unsigned long long pt_get_wait_limit_ns();

// D (bf16, [M,N], row stride ldd, at element offset d_offset of the symmetric data region) = sum over the `world` ranks of
// op(A) op(B); layouts as pt_gemm_bf16 (a_mn, b_mn). buf_ptrs / flag_ptrs: peer-mapped bases of the data and flag regions
// mc_ptr: multicast mapping of the data region (NVSwitch reduction) or null (plain peer loads/stores).
// (flag region >= 16 KiB + 4*(1024*2*8 + 1024*2) bytes, zero-initialised once). The epoch of the call comes from the
// workspace's call counter in device memory, so all ranks must issue the same sequence of collective calls on the
// workspace. All ranks must call with the same shapes and the same `clusters_cap` (the number of CTA
// pairs of the grid; tile ownership depends on it). clusters_cap <= 0: launch nothing and return this device's maximum. Returns -5 if CTA pairs cannot be scheduled,
// -12 if the problem has more than 1024 output tiles of 256x256.
extern "C" int pt_gemm_allreduce_bf16(const void* A, const void* B, void* const* buf_ptrs, void* const* flag_ptrs,
                                      void* mc_ptr, long long d_offset, int M, int N, int K, long long lda, long long ldb, long long ldd,
                                      int a_mn, int b_mn, int rank, int world, int clusters_cap,
                                      cudaStream_t stream) {
  using namespace pt;
  using namespace pt::gemm_ar;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (world < 1 || world > MAX_RANKS || (lda % 8) || (ldb % 8) || (ldd % 8) || (N % 8) || (d_offset % 8) ||
      (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -10;
  CUtensorMap ma, mb;
  int rc;
  rc = a_mn ? make_bf16_map_2d(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 64, BK)
            : make_bf16_map_2d(&ma, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, BM);
  if (rc) return rc * 10 - 1;
  rc = b_mn ? make_bf16_map_2d(&mb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, BK)
            : make_bf16_map_2d(&mb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, BN_HALF);
  if (rc) return rc * 10 - 2;
  Peers peers;
  for (int q = 0; q < MAX_RANKS; ++q) {
    peers.buf[q] = q < world ? buf_ptrs[q] : nullptr;
    peers.flags[q] = q < world ? reinterpret_cast<unsigned int*>(flag_ptrs[q]) : nullptr;
  }
  KernelStatus* st = reinterpret_cast<KernelStatus*>(pt_status_word());
  const unsigned long long wait_ns = pt_get_wait_limit_ns();
  if (!a_mn && !b_mn) return launch<false, false>(ma, mb, peers, mc_ptr, d_offset, M, N, K, ldd, rank, world, wait_ns, clusters_cap, st, stream);
  if (!a_mn && b_mn) return launch<false, true>(ma, mb, peers, mc_ptr, d_offset, M, N, K, ldd, rank, world, wait_ns, clusters_cap, st, stream);
  if (a_mn && b_mn) return launch<true, true>(ma, mb, peers, mc_ptr, d_offset, M, N, K, ldd, rank, world, wait_ns, clusters_cap, st, stream);
  return launch<true, false>(ma, mb, peers, mc_ptr, d_offset, M, N, K, ldd, rank, world, wait_ns, clusters_cap, st, stream);
}

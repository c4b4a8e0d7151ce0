// bf16 GEMM for sm_100a on CTA pairs (tcgen05 cta_group::2): D[M,N] = op(A) * op(B), fp32 accumulate in TMEM.
//
// Same contract and operand layouts as gemm_tcgen05.cu, but two CTAs (a cluster of 2 on neighbouring SMs)
// cooperate on one 256x256 output tile: each CTA loads its own 128 rows of A and its own 128 columns of
// B -- with plain, non-multicast TMA loads -- and one thread of the leader CTA issues a 256-row MMA that
// reads both CTAs' shared memory and writes both CTAs' tensor memory. Per output element this moves a
// third less operand data from L2 into shared memory than the single-CTA 128x256 tile (each B half is
// fetched once per pair instead of once per CTA), which is what the single-CTA kernel is limited by.
//
// Synchronisation between the two CTAs:
//   full[s]       lives in the leader; the leader's producer arms it with the bytes of BOTH CTAs, the
//                 peer's TMA loads credit their bytes to it (cta_group::2 form of the load).
//   empty[s]      one per CTA; the leader's MMA thread commits to both after the MMAs that read stage s.
//   tmem_full[a]  one per CTA; committed to both after the last k-block of a tile.
//   tmem_empty[a] lives in the leader; the four epilogue warps of each CTA arrive on it (the peer remotely).
// Every wait is bounded; a cluster barrier at start (barriers initialised) and at the end (nobody may
// exit while its partner can still touch its shared memory) brackets the kernel.
//
// Epilogue. Each of the four epilogue warps drains its 32 accumulator rows in chunks of 128 bytes per row
// (64 bf16 or 32 fp32 columns), writes a chunk into a 128B-swizzled 4 KiB staging buffer of its own (two per
// warp) and one lane hands it to TMA: a tiled store for bf16 / fp32 outputs, a tiled reduce-add for the
// "accumulate into an fp32 destination" mode, so the weight-gradient GEMMs never read their destination into
// the SM. TMA clips rows and columns beyond M and N. The older epilogue (each thread storing its own row with
// 16-byte stores, read-modify-write for the accumulate mode) is kept as a template variant.
//
// Fused epilogues (forward GEMMs X W^T with bf16 output only):
//   SwiGLU  W is the packed [gate; up] weight [2I, K]. The leader CTA loads 128 gate rows, its partner the 128 up rows of
//           the same indices, so accumulator columns 0..127 / 128..255 of a tile are gate / up pre-activations of the
//           same 128 hidden units. The epilogue stores both (the backward needs them) and silu(gate) * up to a second
//           output, which replaces the separate activation kernel and its pass over the [T, 2I] tensor.
//   RoPE    the output is the packed q|k|v activation; columns of the rotated heads (a prefix) are rotated in fp32 with
//           the cos/sin of the row's position before the single rounding to bf16 (NeoX pairing j <-> j + d/2, which
//           lies inside one 64-column chunk for d = 64 and inside one pair of chunks for d = 128).
// Epilogues that READ a second operand (the epilogue warps fetch its tile with TMA into their staging buffers while the
// accumulator is still being computed, combine it in place and hand the same buffers to the TMA store):
//   ADD         forward layout: D = A B^T + R with R a bf16 [M, N] tensor (the residual stream): the separate add kernel
//               and its pass over three [T, H] tensors disappear.
//   SWIGLU_BWD  dgrad layout (dY W): the accumulator is da = dL/d(silu(gate) * up) for 64 hidden units at a time; the
//               epilogue loads the matching gate and up pre-activations from the packed [M, 2I] tensor and stores
//               dgate = da * up * silu'(gate) and dup = da * silu(gate) into a packed [M, 2I] gradient. da itself is
//               never written, and the SwiGLU-backward kernel with its five passes over [T, I] is gone. This variant
//               runs with five operand stages because each epilogue warp needs four staging buffers.
#include "common.cuh"
#include "tensormap.cuh"

extern "C" void pt_count_launches(int n);

namespace pt {
namespace gemm_pair {

constexpr int BM = 128;        // rows of A per CTA (256 per pair)
constexpr int BN_HALF = 128;   // columns of B per CTA (256 per pair)
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK * 2;        // 16 KiB
constexpr int B_BYTES = BN_HALF * BK * 2;   // 16 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int STAGING_BYTES = 4 * 2 * 4096;   // 4 epilogue warps x 2 buffers of [32 rows][128 B]
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STAGING_BYTES + 1024;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr unsigned KERNEL_ID = 2;

enum OutMode { OUT_BF16 = 0, OUT_F32_ACC = 1, OUT_F32 = 2 };
enum Epilogue { EPI_NONE = 0, EPI_SWIGLU = 1, EPI_ROPE64 = 2, EPI_ROPE128 = 3, EPI_ADD = 4, EPI_SWIGLU_BWD = 5, EPI_CE = 6 };
// operand stages and staging buffers per epilogue warp of each variant (see the smem budget in launch())
__host__ __device__ constexpr int stages_of(int epi) { return epi == EPI_SWIGLU_BWD ? 5 : 6; }
__host__ __device__ constexpr int staging_bufs_of(int epi) { return epi == EPI_SWIGLU_BWD ? 4 : 2; }
__host__ __device__ constexpr int smem_bytes_of(int epi) {
  return stages_of(epi) * STAGE_BYTES + 4 * staging_bufs_of(epi) * 4096 + 1024;
}

struct EpiArgs {
  int inter;              // SwiGLU: I (the weight has 2 I rows, the second output I columns)
  const float* cosT;      // RoPE: fp32 [S, d/2] tables
  const float* sinT;
  int seq;                // RoPE: row r is at position r % seq
  int rot_cols;           // RoPE: columns [0, rot_cols) are rotated (rotated heads x d)
  int group_m;            // tile numbering: rows of tiles per group (all epilogues)
  // cross-entropy statistics (EPI_CE): per row and per 256-column tile the maximum and the sum of exp(logit - maximum)
  // of the ROUNDED logits go to ce_part[row * ce_tiles + n_blk]; the logit of the row's target column goes to ce_tgt[row]
  float2* ce_part;
  float* ce_tgt;
  const long long* ce_targets;
  long long ce_vocab_start;
  int ce_tiles;
};

struct Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t epi_load[4][2];    // per epilogue warp and buffer pair: the TMA loads of the second operand (ADD / SWIGLU_BWD)
  uint32_t tmem_base;
  int abort_flag;
};

// Tiles are numbered in groups of `group_m` rows of tiles, column by column inside a group, so that the CTA pairs that run
// at the same time (consecutive tile numbers) share few A row panels and few B column panels in L2.
__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int group_m, int& m_blk, int& n_blk) {
  const int per_group = group_m * num_n;
  const int group = t / per_group;
  const int first_m = group * group_m;
  const int gsize = min(num_m - first_m, group_m);
  const int r = t - group * per_group;
  m_blk = first_m + r % gsize;
  n_blk = r / gsize;
}

__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* m, const void* smem_src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
// byte offset of 16-byte unit u of row r in a [rows][128 B] tile stored with the 128-byte swizzle
__device__ __forceinline__ uint32_t sw128_unit(int r, int u) { return (uint32_t)(r * 128 + ((u ^ (r & 7)) << 4)); }

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// N is the number of output columns, except for EPI_SWIGLU where it is I (tiles pair 128 gate with 128 up columns).
template <bool A_MN, bool B_MN, int OUT_MODE, bool EPI_TMA, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const __grid_constant__ CUtensorMap tma_d, const __grid_constant__ CUtensorMap tma_h,
                 void* __restrict__ Dptr, int M, int N, int K, long long ldd, KernelStatus* status, EpiArgs ea) {
  static_assert(EPI == EPI_NONE || (EPI_TMA && !A_MN && OUT_MODE == OUT_BF16 && B_MN == (EPI == EPI_SWIGLU_BWD)),
                "fused epilogues: bf16 output; forward layout, except the SwiGLU backward which rides on the dgrad layout");
  constexpr int STAGES = stages_of(EPI);          // shadows the namespace constant: the variants differ in their smem split
  pdl_launch_dependents();
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
  const int num_n = (EPI == EPI_SWIGLU) ? (N + BN_HALF - 1) / BN_HALF : (N + BN - 1) / BN;
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
      for (int q = 0; q < 4; ++q) mbar_init(&bars.epi_load[q][s], 1);
    }
    bars.abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
    if (EPI_TMA) tma_prefetch_desc(&tma_d);
    if (EPI == EPI_SWIGLU || EPI == EPI_ADD || EPI == EPI_SWIGLU_BWD) tma_prefetch_desc(&tma_h);
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
  pdl_wait();                      // the prologue above ran under the predecessor's tail; its results are needed from here on
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
        tile_coords(t, num_m, num_n, ea.group_m, m_blk, n_blk);
        const int row0 = m_blk * 2 * BM + (int)rank * BM;          // this CTA's rows of A
        // this CTA's columns of B (SwiGLU: gate rows for the leader, the up rows of the same units for its partner)
        const int col0 = (EPI == EPI_SWIGLU) ? n_blk * BN_HALF + (int)rank * ea.inter : n_blk * BN + (int)rank * BN_HALF;
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
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int quarter = warp & 3;
    bool ok = true;
    int local = 0;
    if constexpr (EPI == EPI_ADD || EPI == EPI_SWIGLU_BWD) {
      // ---- epilogues with a second operand: chunk c of a tile = 64 accumulator columns of this warp's 32 rows
      constexpr int NBUF = staging_bufs_of(EPI);              // 2: one buffer per chunk; 4: (gate, up) per chunk
      constexpr int PER = NBUF / 2;                           // buffers per chunk
      constexpr int NCH = BN / 64;
      uint8_t* stg = smem + STAGES * STAGE_BYTES + quarter * (NBUF * 4096);
      uint32_t ld_phase[2] = {0, 0};
      int seq = 0;                                            // chunks handled so far: chunk `seq` uses buffer set seq & 1
      // Load the second operand of chunk (tile t, c) into buffer set `set`. The previous user of that set is the chunk before
      // the current one; its TMA store, issued a moment ago, must have finished reading the buffers.
      auto issue_load = [&](int t, int c, int set) {
        if (lane != 0) return;
        int m_blk, n_blk;
        tile_coords(t, num_m, num_n, ea.group_m, m_blk, n_blk);
        const int row0 = m_blk * 2 * BM + (int)rank * BM + quarter * 32;
        const int col0 = n_blk * BN + c * 64;
        tma_store_wait_read<0>();        // (overlaps the tensor-memory load issued just before)
        uint8_t* b0 = stg + set * PER * 4096;
        if (row0 < M && col0 < N) {
          mbar_expect_tx(&bars.epi_load[quarter][set], PER * 4096);
          tma_load_2d(b0, &tma_h, &bars.epi_load[quarter][set], col0, row0);
          if (EPI == EPI_SWIGLU_BWD) tma_load_2d(b0 + 4096, &tma_h, &bars.epi_load[quarter][set], ea.inter + col0, row0);
        } else {
          mbar_arrive(&bars.epi_load[quarter][set]);          // nothing to fetch: complete the phase by hand
        }
      };
      if (cluster_id < num_tiles) issue_load(cluster_id, 0, 0);
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++local) {
        int m_blk, n_blk;
        tile_coords(t, num_m, num_n, ea.group_m, m_blk, n_blk);
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&bars.tmem_full[acc], acc_phase, abort_flag)) {
          if (lane == 0) report_error(status, KERNEL_ID, 4);
          ok = false;
          break;
        }
        tcgen05_fence_after();
        const int row0 = m_blk * 2 * BM + (int)rank * BM + quarter * 32;
        const uint32_t t_row = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
        for (int c = 0; c < NCH; ++c, ++seq) {
          const int set = seq & 1;
          uint32_t v[64];
          tmem_ld_32x32b_x32_at(t_row + c * 64, v, 0);
          tmem_ld_32x32b_x32_at(t_row + c * 64 + 32, v, 32);
          // the operand of the next chunk (of this tile or of the next one) travels while this one is combined
          if (c + 1 < NCH) issue_load(t, c + 1, set ^ 1);
          else if (t + num_clusters < num_tiles) issue_load(t + num_clusters, 0, set ^ 1);
          tmem_ld_wait();
          if (!mbar_wait(&bars.epi_load[quarter][set], ld_phase[set], abort_flag)) {
            if (lane == 0) report_error(status, KERNEL_ID, 5);
            ok = false;
            break;
          }
          ld_phase[set] ^= 1;
          uint8_t* b0 = stg + set * PER * 4096;
          const int col0 = n_blk * BN + c * 64;
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const uint32_t off = sw128_unit(lane, u);
            uint4 q0 = *reinterpret_cast<const uint4*>(b0 + off);
            uint32_t* w0 = reinterpret_cast<uint32_t*>(&q0);
            if constexpr (EPI == EPI_ADD) {
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 r = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w0[e]));
                w0[e] = pack_bf16(__uint_as_float(v[8 * u + 2 * e]) + r.x, __uint_as_float(v[8 * u + 2 * e + 1]) + r.y);
              }
              *reinterpret_cast<uint4*>(b0 + off) = q0;
            } else {
              uint4 q1 = *reinterpret_cast<const uint4*>(b0 + 4096 + off);
              uint32_t* w1 = reinterpret_cast<uint32_t*>(&q1);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w0[e]));
                const float2 up = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w1[e]));
                const float da0 = __uint_as_float(v[8 * u + 2 * e]), da1 = __uint_as_float(v[8 * u + 2 * e + 1]);
                const float s0 = __fdividef(1.f, 1.f + ex2_approx(-g.x * 1.4426950408889634f));
                const float s1 = __fdividef(1.f, 1.f + ex2_approx(-g.y * 1.4426950408889634f));
                w0[e] = pack_bf16(da0 * up.x * (s0 * (1.f + g.x * (1.f - s0))), da1 * up.y * (s1 * (1.f + g.y * (1.f - s1))));
                w1[e] = pack_bf16(da0 * g.x * s0, da1 * g.y * s1);
              }
              *reinterpret_cast<uint4*>(b0 + off) = q0;
              *reinterpret_cast<uint4*>(b0 + 4096 + off) = q1;
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (row0 < M && col0 < N) {
              tma_store_2d(&tma_d, b0, col0, row0);
              if (EPI == EPI_SWIGLU_BWD) tma_store_2d(&tma_d, b0 + 4096, ea.inter + col0, row0);
            }
            tma_store_commit();
          }
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&bars.tmem_empty[acc]), 0));
      }
      if (lane == 0) tma_store_wait<0>();
    } else if constexpr (EPI != EPI_NONE) {
      uint8_t* stg = smem + STAGES * STAGE_BYTES + quarter * (2 * 4096);
      int buf = 0;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++local) {
        int m_blk, n_blk;
        tile_coords(t, num_m, num_n, ea.group_m, m_blk, n_blk);
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&bars.tmem_full[acc], acc_phase, abort_flag)) {
          if (lane == 0) report_error(status, KERNEL_ID, 4);
          ok = false;
          break;
        }
        tcgen05_fence_after();
        const int row0 = m_blk * 2 * BM + (int)rank * BM + quarter * 32;      // first of this warp's 32 rows
        const uint32_t t_row = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN;
        // 64 bf16 of this lane's row (packed in q[32]) -> swizzled staging buffer -> TMA store at (col0, row0)
        auto stage_store = [&](const uint32_t (&q)[32], const CUtensorMap* map, int col0) {
          if (lane == 0) tma_store_wait_read<1>();        // the store issued two chunks ago has finished reading this buffer
          __syncwarp();
          uint8_t* dst = stg + buf * 4096;
#pragma unroll
          for (int u = 0; u < 8; ++u)
            *reinterpret_cast<uint4*>(dst + sw128_unit(lane, u)) = make_uint4(q[4 * u], q[4 * u + 1], q[4 * u + 2], q[4 * u + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (row0 < M) tma_store_2d(map, dst, col0, row0);
            tma_store_commit();
          }
          buf ^= 1;
        };
        if constexpr (EPI == EPI_SWIGLU) {
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            uint32_t g[64], u[64];
            tmem_ld_32x32b_x32_at(t_row + c * 64, g, 0);
            tmem_ld_32x32b_x32_at(t_row + c * 64 + 32, g, 32);
            tmem_ld_32x32b_x32_at(t_row + BN_HALF + c * 64, u, 0);
            tmem_ld_32x32b_x32_at(t_row + BN_HALF + c * 64 + 32, u, 32);
            tmem_ld_wait();
            uint32_t qg[32], qu[32], qh[32];
#pragma unroll
            for (int e = 0; e < 64; e += 2) {
              qg[e >> 1] = pack_bf16(__uint_as_float(g[e]), __uint_as_float(g[e + 1]));
              qu[e >> 1] = pack_bf16(__uint_as_float(u[e]), __uint_as_float(u[e + 1]));
              // the activation is computed from the ROUNDED pre-activations, which is what the backward will read
              const float2 gr = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qg[e >> 1]));
              const float2 ur = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qu[e >> 1]));
              const float h0 = gr.x * __fdividef(1.f, 1.f + ex2_approx(-gr.x * 1.4426950408889634f)) * ur.x;
              const float h1 = gr.y * __fdividef(1.f, 1.f + ex2_approx(-gr.y * 1.4426950408889634f)) * ur.y;
              qh[e >> 1] = pack_bf16(h0, h1);
            }
            const int unit0 = n_blk * BN_HALF + c * 64;
            stage_store(qg, &tma_d, unit0);
            stage_store(qu, &tma_d, ea.inter + unit0);
            stage_store(qh, &tma_h, unit0);
          }
        } else if constexpr (EPI == EPI_CE) {
          // LM-head logits tile: store it, and keep per row the running maximum and the sum of exponentials over the
          // tile's 256 columns (online, chunk by chunk) of the values as stored (bf16), plus the target's logit
          const int row = row0 + lane;
          const long long tcol = (row < M ? ea.ce_targets[row] : -1) - ea.ce_vocab_start;     // column of the target in this shard
          float m_run = -INFINITY, s_run = 0.f;
#pragma unroll 1
          for (int c = 0; c < BN / 64; ++c) {
            uint32_t v[64];
            tmem_ld_32x32b_x32_at(t_row + c * 64, v, 0);
            tmem_ld_32x32b_x32_at(t_row + c * 64 + 32, v, 32);
            tmem_ld_wait();
            const int col0 = n_blk * BN + c * 64;
            uint32_t q[32];
            float cm = -INFINITY;
#pragma unroll
            for (int e = 0; e < 64; e += 2) {
              q[e >> 1] = pack_bf16(__uint_as_float(v[e]), __uint_as_float(v[e + 1]));
              const float2 r = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q[e >> 1]));
              v[e] = __float_as_uint(col0 + e < N ? r.x : -INFINITY);
              v[e + 1] = __float_as_uint(col0 + e + 1 < N ? r.y : -INFINITY);
              cm = fmaxf(cm, fmaxf(__uint_as_float(v[e]), __uint_as_float(v[e + 1])));
            }
            if (col0 < N) {
              const float nm = fmaxf(m_run, cm);
              float acc = 0.f;
#pragma unroll
              for (int e = 0; e < 64; ++e) acc += ex2_approx((__uint_as_float(v[e]) - nm) * 1.4426950408889634f);
              s_run = s_run * ex2_approx((m_run - nm) * 1.4426950408889634f) + acc;
              m_run = nm;
              if (tcol >= col0 && tcol < col0 + 64 && tcol < N && row < M) {     // (a target beyond N belongs to another shard)
                float tv = 0.f;
#pragma unroll
                for (int e = 0; e < 64; ++e) tv = ((long long)(col0 + e) == tcol) ? __uint_as_float(v[e]) : tv;
                ea.ce_tgt[row] = tv;
              }
              stage_store(q, &tma_d, col0);
            }
          }
          if (row < M) ea.ce_part[(long long)row * ea.ce_tiles + n_blk] = make_float2(m_run, s_run);
        } else {
          constexpr int HD = (EPI == EPI_ROPE64) ? 64 : 128;          // head dim = columns handled per iteration
          const int row = row0 + lane;
          const int pos = (row < M ? row : 0) % ea.seq;
          const float* cos_row = ea.cosT + (long long)pos * (HD / 2);
          const float* sin_row = ea.sinT + (long long)pos * (HD / 2);
#pragma unroll 1
          for (int c = 0; c < BN / HD; ++c) {
            uint32_t v[HD];
#pragma unroll
            for (int h = 0; h < HD / 32; ++h) tmem_ld_32x32b_x32_at(t_row + c * HD + h * 32, v, h * 32);
            tmem_ld_wait();
            const int col0 = n_blk * BN + c * HD;
            if (col0 < ea.rot_cols) {
#pragma unroll
              for (int jj = 0; jj < HD / 2; jj += 4) {
                const float4 cs = __ldg(reinterpret_cast<const float4*>(cos_row + jj));
                const float4 sn = __ldg(reinterpret_cast<const float4*>(sin_row + jj));
                const float csv[4] = {cs.x, cs.y, cs.z, cs.w}, snv[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float a = __uint_as_float(v[jj + i]), b = __uint_as_float(v[jj + i + HD / 2]);
                  v[jj + i] = __float_as_uint(a * csv[i] - b * snv[i]);
                  v[jj + i + HD / 2] = __float_as_uint(b * csv[i] + a * snv[i]);
                }
              }
            }
#pragma unroll
            for (int part = 0; part < HD / 64; ++part) {
              uint32_t q[32];
#pragma unroll
              for (int e = 0; e < 64; e += 2)
                q[e >> 1] = pack_bf16(__uint_as_float(v[part * 64 + e]), __uint_as_float(v[part * 64 + e + 1]));
              if (col0 + part * 64 < N) stage_store(q, &tma_d, col0 + part * 64);
            }
          }
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&bars.tmem_empty[acc]), 0));
      }
      if (lane == 0) tma_store_wait<0>();
    } else if constexpr (EPI_TMA) {
      constexpr int CH_COLS = (OUT_MODE == OUT_BF16) ? 64 : 32;      // columns per 128-byte chunk row

      constexpr int NCH = BN / CH_COLS;
      constexpr int CH_REGS = (OUT_MODE == OUT_BF16) ? 64 : 32;      // accumulator registers per chunk
      uint8_t* stg = smem + STAGES * STAGE_BYTES + quarter * (2 * 4096);
      int buf = 0;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++local) {
        int m_blk, n_blk;
        tile_coords(t, num_m, num_n, ea.group_m, m_blk, n_blk);
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&bars.tmem_full[acc], acc_phase, abort_flag)) {
          if (lane == 0) report_error(status, KERNEL_ID, 4);
          ok = false;
          break;
        }
        tcgen05_fence_after();
        const int row0 = m_blk * 2 * BM + (int)rank * BM + quarter * 32;      // first of this warp's 32 rows
        const uint32_t t_row = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN;
        uint32_t r[2][CH_REGS];
        auto load_chunk = [&](int c, uint32_t (&dst)[CH_REGS]) {
#pragma unroll
          for (int h = 0; h < CH_REGS / 32; ++h) tmem_ld_32x32b_x32_at(t_row + c * CH_COLS + h * 32, dst, h * 32);
        };
        load_chunk(0, r[0]);
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          tmem_ld_wait();
          if (c + 1 < NCH) load_chunk(c + 1, r[(c + 1) & 1]);
          const uint32_t (&v)[CH_REGS] = r[c & 1];
          if (lane == 0) tma_store_wait_read<1>();        // the store issued two chunks ago has finished reading this buffer
          __syncwarp();
          uint8_t* dst = stg + buf * 4096;
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            uint4 q;
            if (OUT_MODE == OUT_BF16) {
              q.x = pack_bf16(__uint_as_float(v[8 * u + 0]), __uint_as_float(v[8 * u + 1]));
              q.y = pack_bf16(__uint_as_float(v[8 * u + 2]), __uint_as_float(v[8 * u + 3]));
              q.z = pack_bf16(__uint_as_float(v[8 * u + 4]), __uint_as_float(v[8 * u + 5]));
              q.w = pack_bf16(__uint_as_float(v[8 * u + 6]), __uint_as_float(v[8 * u + 7]));
            } else {
              q = make_uint4(v[(4 * u + 0) % CH_REGS], v[(4 * u + 1) % CH_REGS], v[(4 * u + 2) % CH_REGS], v[(4 * u + 3) % CH_REGS]);
            }
            *reinterpret_cast<uint4*>(dst + sw128_unit(lane, u)) = q;
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const int col0 = n_blk * BN + c * CH_COLS;
            if (row0 < M && col0 < N) {
              if (OUT_MODE == OUT_F32_ACC) tma_reduce_add_2d(&tma_d, dst, col0, row0);
              else tma_store_2d(&tma_d, dst, col0, row0);
            }
            tma_store_commit();
          }
          buf ^= 1;
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&bars.tmem_empty[acc]), 0));
      }
      if (lane == 0) tma_store_wait<0>();
    } else {
    for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++local) {
      int m_blk, n_blk;
      tile_coords(t, num_m, num_n, ea.group_m, m_blk, n_blk);
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
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&bars.tmem_empty[acc]), 0));
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
}

static int g_group_m = 8;   // rows of 256-row tiles per group; measured on the model's shapes: 8 and 16 beat 4 by ~1 %, 1 is worst

template <bool A_MN, bool B_MN, int OUT_MODE, bool EPI_TMA, int EPI = EPI_NONE>
static int launch(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& md, void* D, int M, int N, int K,
                  long long ldd, KernelStatus* status, cudaStream_t stream, const CUtensorMap* mh = nullptr,
                  EpiArgs ea = EpiArgs{}) {
  auto kern = gemm_pair_kernel<A_MN, B_MN, OUT_MODE, EPI_TMA, EPI>;
  static int max_clusters = 0;
  if (max_clusters == 0) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes_of(EPI)) != cudaSuccess) return -3;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2, 1, 1);
    cfg.blockDim = dim3(NUM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem_bytes_of(EPI);
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
  const int n_tiles = (EPI == EPI_SWIGLU) ? (N + BN_HALF - 1) / BN_HALF : (N + BN - 1) / BN;
  const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * n_tiles;
  const int clusters = tiles < max_clusters ? tiles : max_clusters;
  ea.group_m = g_group_m;
  const cudaError_t err = launch_pdl(kern, dim3(2 * clusters), dim3(NUM_THREADS), smem_bytes_of(EPI), stream, ma, mb, md,
                                     mh ? *mh : md, D, M, N, K, ldd, status, ea);
  pt_count_launches(1);
  return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? 0 : -4;
}

}  // namespace gemm_pair
}  // namespace pt

extern "C" void pt_gemm_set_group_m(int g) { pt::gemm_pair::g_group_m = g < 1 ? 1 : g; }
extern "C" int pt_gemm_get_group_m() { return pt::gemm_pair::g_group_m; }

// 1 (default): epilogue through shared memory and TMA store / reduce-add; 0: per-thread 16-byte stores.
static int g_tma_epilogue = 1;
extern "C" void pt_gemm_set_tma_epilogue(int on) { g_tma_epilogue = on; }
extern "C" int pt_gemm_get_tma_epilogue() { return g_tma_epilogue; }

// Same contract as pt_gemm_bf16 (gemm_tcgen05.cu). Returns -5 when CTA pairs cannot be scheduled.
extern "C" int pt_gemm_bf16_pair(const void* A, const void* B, void* D, int M, int N, int K, long long lda,
                                 long long ldb, long long ldd, int a_mn, int b_mn, int out_mode, void* status,
                                 cudaStream_t stream) {
  using namespace pt;
  using namespace pt::gemm_pair;
  CUtensorMap ma, mb;
  int rc;
  rc = a_mn ? make_bf16_map_2d(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 64, BK)
            : make_bf16_map_2d(&ma, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, BM);
  if (rc) return rc * 10 - 1;    // -21: tensor map of A could not be encoded
  rc = b_mn ? make_bf16_map_2d(&mb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, BK)
            : make_bf16_map_2d(&mb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, BN_HALF);
  if (rc) return rc * 10 - 2;    // -22: tensor map of B could not be encoded
  CUtensorMap md = ma;           // unused by the per-thread epilogue
  const bool epi_tma = g_tma_epilogue != 0;
  if (epi_tma) {
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)M};
    uint64_t strides[1] = {(uint64_t)ldd};
    uint32_t box_bf16[2] = {64, 32}, box_f32[2] = {32, 32};
    rc = out_mode == OUT_BF16 ? make_bf16_map(&md, D, 2, dims, strides, box_bf16) : make_f32_map(&md, D, 2, dims, strides, box_f32);
    if (rc) return rc * 10 - 3;  // -23: tensor map of D could not be encoded
  }
  KernelStatus* st = reinterpret_cast<KernelStatus*>(status);
#define PT_GEMM_CASE(AM, BMN, OM)                                                                             \
  if (a_mn == AM && b_mn == BMN && out_mode == OM)                                                            \
    return epi_tma ? launch<AM, BMN, OM, true>(ma, mb, md, D, M, N, K, ldd, st, stream)                       \
                   : launch<AM, BMN, OM, false>(ma, mb, md, D, M, N, K, ldd, st, stream);
  PT_GEMM_CASE(0, 0, 0) PT_GEMM_CASE(0, 0, 1) PT_GEMM_CASE(0, 0, 2)
  PT_GEMM_CASE(0, 1, 0) PT_GEMM_CASE(0, 1, 1) PT_GEMM_CASE(0, 1, 2)
  PT_GEMM_CASE(1, 1, 0) PT_GEMM_CASE(1, 1, 1) PT_GEMM_CASE(1, 1, 2)
  PT_GEMM_CASE(1, 0, 0) PT_GEMM_CASE(1, 0, 1) PT_GEMM_CASE(1, 0, 2)
#undef PT_GEMM_CASE
  return -11;
}

// Forward GEMM D[M, N] = A[M, K] B[N, K]^T (bf16) with a fused epilogue; requirements as pt_gemm_bf16 plus:
//   epi 1 (SwiGLU): B is [2 I, K] (gate rows, then up rows), D is [M, 2 I] (ldd), H is [M, I] bf16 (ldh, 16-byte aligned,
//                   ldh % 8 == 0), I % 128 == 0; N is ignored.
//   epi 2 (RoPE):   D is the packed q|k|v activation [M, N]; head_dim 64 or 128; columns [0, rot_heads * head_dim) are
//                   rotated with cosT/sinT (fp32 [seq, head_dim / 2], 16-byte aligned) at position row % seq.
//   epi 4 (ADD):    D = A B^T + H with H a bf16 [M, N] tensor (ldh); N % 8 == 0.
//   epi 5 (SwiGLU backward, dgrad layout): A is dY [M, K], B is the down-projection weight stored [K, I] (ldb), so the
//                   accumulator is da [M, I]; H is the packed pre-activation [M, 2 I] (ldh), D the packed gradient [M, 2 I]
//                   (ldd): D[:, :I] = da * up * silu'(gate), D[:, I:] = da * silu(gate). inter = I, I % 64 == 0; N is ignored.
// Returns 1 (nothing launched) when the shape is not covered, so that the caller can run the unfused kernels.
extern "C" int pt_gemm_bf16_fused(const void* A, const void* B, void* D, int M, int N, int K, long long lda, long long ldb,
                                  long long ldd, int epi, void* H, long long ldh, int inter, const float* cosT,
                                  const float* sinT, int seq, int rot_heads, int head_dim, void* status,
                                  cudaStream_t stream) {
  using namespace pt;
  using namespace pt::gemm_pair;
  if (!g_tma_epilogue) return 1;
  if ((lda % 8) || (ldb % 8) || (ldd % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (reinterpret_cast<uintptr_t>(D) & 15))
    return -10;
  EpiArgs ea{};
  int n_out = N;
  if (epi == EPI_SWIGLU) {
    if (inter <= 0 || inter % BN_HALF || H == nullptr || (ldh % 8) || (reinterpret_cast<uintptr_t>(H) & 15)) return 1;
    ea.inter = inter;
    n_out = 2 * inter;
  } else if (epi == EPI_ADD) {
    if (H == nullptr || (ldh % 8) || (reinterpret_cast<uintptr_t>(H) & 15) || (N % 8)) return 1;
  } else if (epi == EPI_SWIGLU_BWD) {
    if (inter <= 0 || inter % 64 || H == nullptr || (ldh % 8) || (reinterpret_cast<uintptr_t>(H) & 15)) return 1;
    ea.inter = inter;
    n_out = 2 * inter;
  } else if (epi == 2) {
    if ((head_dim != 64 && head_dim != 128) || seq <= 0 || cosT == nullptr || sinT == nullptr ||
        (reinterpret_cast<uintptr_t>(cosT) & 15) || (reinterpret_cast<uintptr_t>(sinT) & 15) || rot_heads < 0 ||
        (long long)rot_heads * head_dim > N)
      return 1;
    ea.cosT = cosT;
    ea.sinT = sinT;
    ea.seq = seq;
    ea.rot_cols = rot_heads * head_dim;
  } else {
    return -11;
  }
  if (M <= 0 || n_out <= 0 || K <= 0) return 0;
  CUtensorMap ma, mb, md, mh;
  int rc;
  if ((rc = make_bf16_map_2d(&ma, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, BM))) return rc * 10 - 1;
  if (epi == EPI_SWIGLU_BWD) {
    // B is stored [K, I] (MN-major operand): 64-column x BK-row boxes, as in the plain dgrad GEMM
    if ((rc = make_bf16_map_2d(&mb, B, (uint64_t)inter, (uint64_t)K, (uint64_t)ldb, 64, BK))) return rc * 10 - 2;
  } else {
    if ((rc = make_bf16_map_2d(&mb, B, (uint64_t)K, (uint64_t)n_out, (uint64_t)ldb, BK, BN_HALF))) return rc * 10 - 2;
  }
  if ((rc = make_bf16_map_2d(&md, D, (uint64_t)n_out, (uint64_t)M, (uint64_t)ldd, 64, 32))) return rc * 10 - 3;
  mh = md;
  if ((epi == EPI_ADD || epi == EPI_SWIGLU_BWD) &&
      (rc = make_bf16_map_2d(&mh, H, (uint64_t)n_out, (uint64_t)M, (uint64_t)ldh, 64, 32)))
    return rc * 10 - 4;
  if (epi == EPI_SWIGLU && (rc = make_bf16_map_2d(&mh, H, (uint64_t)inter, (uint64_t)M, (uint64_t)ldh, 64, 32))) return rc * 10 - 4;
  KernelStatus* st = reinterpret_cast<KernelStatus*>(status);
  if (epi == EPI_SWIGLU) return launch<false, false, OUT_BF16, true, EPI_SWIGLU>(ma, mb, md, D, M, inter, K, ldd, st, stream, &mh, ea);
  if (epi == EPI_ADD) return launch<false, false, OUT_BF16, true, EPI_ADD>(ma, mb, md, D, M, N, K, ldd, st, stream, &mh, ea);
  if (epi == EPI_SWIGLU_BWD) return launch<false, true, OUT_BF16, true, EPI_SWIGLU_BWD>(ma, mb, md, D, M, inter, K, ldd, st, stream, &mh, ea);
  if (head_dim == 64) return launch<false, false, OUT_BF16, true, EPI_ROPE64>(ma, mb, md, D, M, N, K, ldd, st, stream, &mh, ea);
  return launch<false, false, OUT_BF16, true, EPI_ROPE128>(ma, mb, md, D, M, N, K, ldd, st, stream, &mh, ea);
}

// LM-head GEMM with the cross-entropy row statistics in its epilogue: D[M, N] = A[M, K] B[N, K]^T (bf16, stored because the
// gradient pass rewrites it in place) and, per row and per 256-column tile, (max, sum exp(logit - max)) of the stored
// values -> part[M, tiles] (tiles = ceil(N / 256)), plus tgt[M] = logit of column targets[row] - vocab_start where that
// column lies in [0, N) (tgt must be zero-filled by the caller: rows whose target belongs to another shard are not
// written). Replaces the separate statistics pass over the logits. Returns 1 when the kernel does not cover the case.
extern "C" int pt_gemm_bf16_ce(const void* A, const void* B, void* D, int M, int N, int K, long long lda, long long ldb,
                               long long ldd, const long long* targets, long long vocab_start, void* part, float* tgt,
                               void* status, cudaStream_t stream) {
  using namespace pt;
  using namespace pt::gemm_pair;
  if (!g_tma_epilogue) return 1;
  if ((lda % 8) || (ldb % 8) || (ldd % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (reinterpret_cast<uintptr_t>(D) & 15) || (reinterpret_cast<uintptr_t>(part) & 7) || (N % 8))
    return -10;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  EpiArgs ea{};
  ea.ce_part = reinterpret_cast<float2*>(part);
  ea.ce_tgt = tgt;
  ea.ce_targets = targets;
  ea.ce_vocab_start = vocab_start;
  ea.ce_tiles = (N + BN - 1) / BN;
  CUtensorMap ma, mb, md;
  int rc;
  if ((rc = make_bf16_map_2d(&ma, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, BM))) return rc * 10 - 1;
  if ((rc = make_bf16_map_2d(&mb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, BN_HALF))) return rc * 10 - 2;
  if ((rc = make_bf16_map_2d(&md, D, (uint64_t)N, (uint64_t)M, (uint64_t)ldd, 64, 32))) return rc * 10 - 3;
  return launch<false, false, OUT_BF16, true, EPI_CE>(ma, mb, md, D, M, N, K, ldd, reinterpret_cast<KernelStatus*>(status), stream,
                                                      &md, ea);
}

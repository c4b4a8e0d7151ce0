// Flash attention forward and backward for sm_100a: tcgen05 MMAs with TMEM accumulators, TMA-fed tiles,
// native GQA, head_dim 64 or 128, causal or full, arbitrary sequence lengths (tails are masked).
//
// Replaces flash_attn_func (FlashAttention-2, mma.sync) at picotron/model.py:33-37,154 and the materialised
// block attention of ring attention (picotron/context_parallel/context_parallel.py:112-155): the same kernels
// compute one ring block when they are given the global log-sum-exp / delta.
//
// Tensors: q [B,Sq,hq,d], k/v [B,Sk,hkv,d] with packed (head, d) and an arbitrary token stride, so slices of
// the packed qkv activation are read in place through 4-D tensor maps {d, head, token, batch}.
// "causal" masks kv index > q index, both counted from the start of their tensors.
//
// Forward, one CTA per (128 query rows, head, batch); two CTAs share an SM so that one CTA's MMAs overlap the
// other's softmax:
//   warp 4    TMA producer: Q once, then K and V blocks through 2-stage rings
//   warp 5    MMA issuer:  S = Q K^T  (TMEM, BN fp32 columns), later  O_j = P_j V_j  (TMEM, d columns)
//   warps 0-3 softmax: thread t owns query row t = TMEM lane t. Online softmax in the exp2 domain, P_j written
//             as bf16 into 128B-swizzled shared memory for the second MMA, the running output kept in
//             registers:  acc = (acc + O_{j-1}) * alpha_j.
//
// Backward, one CTA per (128-key block, kv head, batch) looping over the query heads of the group and the
// query blocks that see this key block:
//   S = Q K^T and dP = dO V^T into TMEM; threads form P = exp2(S*c - lse) and dS = P*(dP - delta)*scale and
//   store both (bf16, swizzled) to shared memory; then dV += P^T dO, dK += dS^T Q (TMEM accumulators that live
//   for the whole CTA) and dQ = dS K, which the threads add to an fp32 workspace with vector reductions.
//   A small kernel computes delta = rowsum(dO*O) beforehand and another converts the fp32 dQ to bf16.
#include "common.cuh"
#include "tensormap.cuh"

extern "C" void pt_count_launches(int n);
extern "C" void* pt_status_word();

namespace pt {
namespace attn {

typedef __nv_bfloat16 bf16;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;
constexpr unsigned KID_FWD = 3, KID_BWD = 4;

inline KernelStatus* status_word_attn() { return reinterpret_cast<KernelStatus*>(pt_status_word()); }

static unsigned long long* g_attn_prof = nullptr;   // device buffer of 16 counters while phase profiling is on

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// byte offset of the 16-byte unit holding columns [8u, 8u+8) of row r inside one [rows][64] bf16 chunk
// stored with the 128-byte swizzle (what TMA writes and UMMA descriptors of layout type SWIZZLE_128B read)
__device__ __forceinline__ uint32_t sw128_offset(int r, int u) { return (uint32_t)(r * 128 + ((u ^ (r & 7)) << 4)); }

// ---------------------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------------------
template <int D, int BN>
struct FwdCfg {
  static constexpr int BM = 128;
  static constexpr int DCH = D / 64;
  static constexpr int Q_BYTES = BM * D * 2;
  static constexpr int KV_BYTES = BN * D * 2;
  static constexpr int P_BYTES = BM * BN * 2;
  static constexpr int STAGES = 2;
  static constexpr int TILES = Q_BYTES + 2 * STAGES * KV_BYTES + P_BYTES;
  static constexpr int SMEM = TILES + 256;            // + barriers; the block starts 1024-byte aligned
  static constexpr int TMEM_COLS = 256;
  static constexpr int S_COL = 0, O_COL = BN;
  static_assert(BN + D <= TMEM_COLS, "TMEM budget");
};

struct FwdBars {
  uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full, s_free, p_ready, o_full;
  uint32_t tmem_base;
  int abort_flag;
};

// K/V may come in up to 8 segments of Sk keys each (the sequence chunks of the context-parallel ranks; a segment's
// tensor map may point into a peer GPU's memory). Keys of segment i precede keys of segment i+1; `causal` applies the
// diagonal mask inside the LAST segment only, every earlier segment is fully visible.
constexpr int MAX_SEGS = 8;
struct KVSegs {
  CUtensorMap k[MAX_SEGS];
  CUtensorMap v[MAX_SEGS];
};

struct AttnParams {
  int B, Sq, Sk, hq, hkv;
  int causal;
  float scale;
  int n_segs;
  unsigned long long* prof;   // optional phase counters (see pt_attention_set_profile); nullptr = not measured
};

// Phase counters of the kernels' consumer threads, in SM clock cycles, summed over all CTAs (thread 0 of each CTA measures):
//   [0] bwd: waiting for S and dP    [1] bwd: TMEM read, exponentials, P/dS stores    [2] bwd: waiting for dQ
//   [3] bwd: dQ drain                [4] bwd: steps          [5] bwd: lifetime of the compute loop    [6] bwd: CTAs
//   [8] fwd: S read + row maximum    [9] fwd: wait for O / rescale   [10] fwd: exponentials + P stores   [11] fwd: blocks
//   [12] fwd: lifetime of the softmax loop   [13] fwd: CTAs   [14] fwd: waiting for S
// Measured only by the PROF instantiations of the kernels, which are launched while a counter buffer is set; the regular
// instantiations contain none of this code.
__device__ __forceinline__ long long prof_clock(bool on) { return on ? clock64() : 0; }

template <int D, int BN, bool PROF>
__global__ void __launch_bounds__(192, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ KVSegs segs, bf16* __restrict__ O,
                float* __restrict__ LSE, AttnParams p, KernelStatus* status) {
  using Cfg = FwdCfg<D, BN>;
  pdl_launch_dependents();
  // no static shared memory in this kernel: the dynamic block starts at the (1024-byte aligned) window base
  extern __shared__ __align__(1024) uint8_t smem[];
  FwdBars& bars = *reinterpret_cast<FwdBars*>(smem + Cfg::TILES);
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Cfg::Q_BYTES;
  uint8_t* sV = sK + Cfg::STAGES * Cfg::KV_BYTES;
  uint8_t* sP = sV + Cfg::STAGES * Cfg::KV_BYTES;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_qb = (p.Sq + Cfg::BM - 1) / Cfg::BM;
  const int qb = num_qb - 1 - (int)(blockIdx.x % num_qb);       // heavy (late) causal blocks first
  const int head = (int)((blockIdx.x / num_qb) % p.hq);
  const int b = (int)(blockIdx.x / (num_qb * p.hq));
  const int kv_head = head / (p.hq / p.hkv);
  const int q0 = qb * Cfg::BM;
  const int bps = (p.Sk + BN - 1) / BN;                              // key blocks per segment
  const int last_end = p.causal ? min(p.Sk, q0 + Cfg::BM) : p.Sk;    // keys of the last segment this tile can see
  const int nblk = (p.n_segs - 1) * bps + (last_end + BN - 1) / BN;

  if (threadIdx.x == 0) {
    mbar_init(&bars.q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars.k_full[s], 1);
      mbar_init(&bars.k_empty[s], 1);
      mbar_init(&bars.v_full[s], 1);
      mbar_init(&bars.v_empty[s], 1);
    }
    mbar_init(&bars.s_full, 1);
    mbar_init(&bars.s_free, 128);
    mbar_init(&bars.p_ready, 128);
    mbar_init(&bars.o_full, 1);
    bars.abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&segs.k[0]);
    tma_prefetch_desc(&segs.v[0]);
  }
  if (warp == 5) {
    tmem_alloc(&bars.tmem_base, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  pdl_wait();                      // barrier init and tensor-memory allocation overlapped the predecessor's tail
  const uint32_t tmem_base = bars.tmem_base;
  volatile int* abort_flag = &bars.abort_flag;

  if (warp == 4) {
    // ------------------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(&bars.q_full, Cfg::Q_BYTES);
#pragma unroll
      for (int c = 0; c < Cfg::DCH; ++c) tma_load_4d(sQ + c * (Cfg::BM * 128), &tm_q, &bars.q_full, c * 64, head, q0, b);
      for (int j = 0; j < nblk; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int seg = j / bps, kv0 = (j - seg * bps) * BN;
        if (!mbar_wait(&bars.k_empty[st], ph ^ 1, abort_flag)) { report_error(status, KID_FWD, 1); break; }
        mbar_expect_tx(&bars.k_full[st], Cfg::KV_BYTES);
#pragma unroll
        for (int c = 0; c < Cfg::DCH; ++c)
          tma_load_4d(sK + st * Cfg::KV_BYTES + c * (BN * 128), &segs.k[seg], &bars.k_full[st], c * 64, kv_head, kv0, b);
        if (!mbar_wait(&bars.v_empty[st], ph ^ 1, abort_flag)) { report_error(status, KID_FWD, 2); break; }
        mbar_expect_tx(&bars.v_full[st], Cfg::KV_BYTES);
#pragma unroll
        for (int c = 0; c < Cfg::DCH; ++c)
          tma_load_4d(sV + st * Cfg::KV_BYTES + c * (BN * 128), &segs.v[seg], &bars.v_full[st], c * 64, kv_head, kv0, b);
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(Cfg::BM, BN, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(Cfg::BM, D, false, true);
      bool ok = mbar_wait(&bars.q_full, 0, abort_flag);
      if (!ok) report_error(status, KID_FWD, 3);
      const uint64_t q_km = make_smem_desc_sw128(smem_u32(sQ), 16, 1024), p_km = make_smem_desc_sw128(smem_u32(sP), 16, 1024);
      // S_{j+1} = Q K_{j+1}^T is issued as soon as the softmax threads have copied S_j out of tensor memory (s_free),
      // i.e. before P_j exists, so it runs under the exponentials of block j instead of after them.
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait(&bars.k_full[st], (j >> 1) & 1, abort_flag)) { report_error(status, KID_FWD, 4); return false; }
        tcgen05_fence_after();
        const uint64_t k_km = make_smem_desc_sw128(smem_u32(sK + st * Cfg::KV_BYTES), 16, 1024);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_bf16(tmem_base + Cfg::S_COL, smem_desc_advance(q_km, (kk >> 2) * (Cfg::BM * 128) + (kk & 3) * 32),
                    smem_desc_advance(k_km, (kk >> 2) * (BN * 128) + (kk & 3) * 32), idesc_s, kk > 0 ? 1u : 0u);
        umma_commit(&bars.s_full);
        umma_commit(&bars.k_empty[st]);
        return true;
      };
      if (ok && nblk > 0) ok = issue_s(0);
      for (int j = 0; j < nblk && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (j + 1 < nblk) {
          if (!mbar_wait(&bars.s_free, j & 1, abort_flag)) { report_error(status, KID_FWD, 10); break; }
          if (!issue_s(j + 1)) break;
        }
        if (!mbar_wait(&bars.p_ready, j & 1, abort_flag)) { report_error(status, KID_FWD, 5); break; }
        if (!mbar_wait(&bars.v_full[st], ph, abort_flag)) { report_error(status, KID_FWD, 6); break; }
        tcgen05_fence_after();
        const uint64_t v_mn = make_smem_desc_sw128(smem_u32(sV + st * Cfg::KV_BYTES), BN * 128, 1024);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)
          umma_bf16(tmem_base + Cfg::O_COL, smem_desc_advance(p_km, (kk >> 2) * (Cfg::BM * 128) + (kk & 3) * 32),
                    smem_desc_advance(v_mn, kk * 2048), idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&bars.o_full);
        umma_commit(&bars.v_empty[st]);
      }
    }
  } else {
    // ------------------------------------------------------------------------------ softmax (warps 0..3)
    // The running output stays in TMEM (the PV MMAs accumulate onto it). Probabilities are taken relative to a
    // reference maximum m_ref that is only moved -- and O rescaled in TMEM -- when the true row maximum has
    // grown by more than 2^8 since the last move, so exp2 never exceeds 256 and the per-block TMEM round trips
    // shrink to one batched read of S.
    const int t = threadIdx.x;                       // query row inside the tile == TMEM lane
    const int row = q0 + t;
    const uint32_t t_lane = tmem_base + (uint32_t(warp * 32) << 16);
    const float sl2 = p.scale * LOG2E;
    constexpr float kRescaleThreshold = 8.f;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    const bool prof_on = PROF && p.prof != nullptr && threadIdx.x == 0;
    long long pacc[4] = {0, 0, 0, 0};
    const long long pstart = prof_clock(prof_on);
    for (int j = 0; j < nblk; ++j) {
      const long long pt0 = prof_clock(prof_on);
      if (!mbar_wait(&bars.s_full, j & 1, abort_flag)) { if (lane == 0) report_error(status, KID_FWD, 7); ok = false; break; }
      tcgen05_fence_after();
      const long long pt1 = prof_clock(prof_on);
      uint32_t s[BN];
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) tmem_ld_32x32b_x32_at(t_lane + Cfg::S_COL + c * 32, s, c * 32);
      tmem_ld_wait();
      tcgen05_fence_before();
      mbar_arrive(&bars.s_free);                                  // S_j is in registers: the next S may overwrite it
      const int seg = j / bps;
      const int col0 = (j - seg * bps) * BN;                      // key index inside its segment
      const bool diag = p.causal && seg == p.n_segs - 1;
      const bool need_mask = (diag && col0 + BN - 1 > q0) || (col0 + BN > p.Sk);
      // four independent running maxima / sums: a single one is a 128-deep chain of dependent instructions
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (need_mask) {
#pragma unroll
        for (int e = 0; e < BN; ++e) {
          const int col = col0 + e;
          if ((diag && col > row) || col >= p.Sk) s[e] = __float_as_uint(-INFINITY);
          mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(s[e]));
        }
      } else {
#pragma unroll
        for (int e = 0; e < BN; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(s[e]));
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_blk = mx * sl2;
      const long long pt2 = prof_clock(prof_on);
      // move the reference? (first finite maximum, or growth beyond the threshold)
      const bool move = m_blk > m_ref + kRescaleThreshold || (m_ref == -INFINITY && m_blk > -INFINITY);
      float alpha = 1.f;
      if (move) {
        alpha = fast_exp2(m_ref - m_blk);            // m_ref == -inf -> 0
        m_ref = m_blk;
        l *= alpha;
      }
      if (j > 0) {
        // P_{j-1} (shared memory) and O (tensor memory) may be touched once the MMA O += P_{j-1} V_{j-1} has completed
        if (!mbar_wait(&bars.o_full, (j - 1) & 1, abort_flag)) { if (lane == 0) report_error(status, KID_FWD, 8); ok = false; break; }
        if (__any_sync(0xffffffffu, move)) {
          tcgen05_fence_after();
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(t_lane + Cfg::O_COL + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
            tmem_st_32x32b_x32(t_lane + Cfg::O_COL + c * 32, r);
          }
          tmem_st_wait();
        }
      }
      const long long pt3 = prof_clock(prof_on);
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      float lsum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t packed[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          const float p0 = fast_exp2(__uint_as_float(s[c * 32 + e]) * sl2 - m_use);       // masked: exp2(-inf) = 0
          const float p1 = fast_exp2(__uint_as_float(s[c * 32 + e + 1]) * sl2 - m_use);
          lsum4[(e >> 1) & 3] += p0 + p1;
          packed[e >> 1] = pack_bf16(p0, p1);
        }
        uint8_t* chunk = sP + ((c * 32) >> 6) * (Cfg::BM * 128);
        const int u0 = ((c * 32) & 63) >> 3;
#pragma unroll
        for (int u = 0; u < 4; ++u)
          *reinterpret_cast<uint4*>(chunk + sw128_offset(t, u0 + u)) =
              make_uint4(packed[4 * u], packed[4 * u + 1], packed[4 * u + 2], packed[4 * u + 3]);
      }
      l += (lsum4[0] + lsum4[1]) + (lsum4[2] + lsum4[3]);
      tcgen05_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(&bars.p_ready);
      if (prof_on) {
        const long long pt4 = clock64();
        pacc[0] += pt2 - pt1; pacc[1] += pt3 - pt2; pacc[2] += pt4 - pt3; pacc[3] += pt1 - pt0;
      }
    }
    if (prof_on) {
      atomicAdd(&p.prof[8], (unsigned long long)pacc[0]);
      atomicAdd(&p.prof[9], (unsigned long long)pacc[1]);
      atomicAdd(&p.prof[10], (unsigned long long)pacc[2]);
      atomicAdd(&p.prof[14], (unsigned long long)pacc[3]);
      atomicAdd(&p.prof[11], (unsigned long long)nblk);
      atomicAdd(&p.prof[12], (unsigned long long)(clock64() - pstart));
      atomicAdd(&p.prof[13], 1ull);
    }
    if (ok && mbar_wait(&bars.o_full, (nblk - 1) & 1, abort_flag)) {
      tcgen05_fence_after();
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      bf16* orow = O + (((long long)b * p.Sq + (row < p.Sq ? row : 0)) * p.hq + head) * D;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_lane + Cfg::O_COL + c * 32, r);
        tmem_ld_wait();
        if (row < p.Sq) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 v = make_uint4(pack_bf16(__uint_as_float(r[8 * u]) * inv_l, __uint_as_float(r[8 * u + 1]) * inv_l),
                                 pack_bf16(__uint_as_float(r[8 * u + 2]) * inv_l, __uint_as_float(r[8 * u + 3]) * inv_l),
                                 pack_bf16(__uint_as_float(r[8 * u + 4]) * inv_l, __uint_as_float(r[8 * u + 5]) * inv_l),
                                 pack_bf16(__uint_as_float(r[8 * u + 6]) * inv_l, __uint_as_float(r[8 * u + 7]) * inv_l));
            reinterpret_cast<uint4*>(orow + c * 32)[u] = v;
          }
        }
      }
      if (row < p.Sq)
        LSE[((long long)b * p.hq + head) * p.Sq + row] = (l > 0.f) ? (m_ref * LN2 + __logf(l)) : -INFINITY;
    } else if (ok && lane == 0) {
      report_error(status, KID_FWD, 9);
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 5) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------------------
// backward helpers: delta = rowsum(dO * O) and fp32 -> bf16 conversion of dQ
// ---------------------------------------------------------------------------------------------------------
// D / 8 threads per (b, s, head) row, 16 bytes of dO and of O per thread, reduced with shuffles inside the group.
template <int D>
__global__ void __launch_bounds__(256)
delta_kernel(const bf16* __restrict__ dO, const bf16* __restrict__ O, float* __restrict__ delta, int B, int S, int h) {
  constexpr int TPR = D / 8;
  pdl_enter();
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)B * S * h;
  const long long rid = tid / TPR;
  const int part = (int)(tid % TPR);
  const long long r = rid < total ? rid : total - 1;            // clamp: every lane takes part in the shuffles
  const uint4 a = *reinterpret_cast<const uint4*>(dO + r * D + part * 8);
  const uint4 o = *reinterpret_cast<const uint4*>(O + r * D + part * 8);
  const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, ow[4] = {o.x, o.y, o.z, o.w};
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 fa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&aw[i]));
    const float2 fo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ow[i]));
    acc += fa.x * fo.x + fa.y * fo.y;
  }
#pragma unroll
  for (int off = TPR / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (part == 0 && rid < total) {
    const int head = (int)(rid % h);
    const long long bs = rid / h;
    const int s = (int)(bs % S), b = (int)(bs / S);
    delta[((long long)b * h + head) * S + s] = acc;
  }
}

// dq_ws: fp32 [B*Sq, hq*d] contiguous -> dq bf16 with token stride dq_row
__global__ void convert_dq_kernel(const float* __restrict__ ws, bf16* __restrict__ dq, long long tokens, int width,
                                  long long dq_row) {
  pdl_enter();
  const long long i4 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i4 >= tokens * width) return;
  const long long tok = i4 / width;
  const int col = (int)(i4 % width);
  const float4 v = *reinterpret_cast<const float4*>(ws + i4);
  uint2 o;
  o.x = pack_bf16(v.x, v.y);
  o.y = pack_bf16(v.z, v.w);
  *reinterpret_cast<uint2*>(dq + tok * dq_row + col) = o;
}

// Same conversion with the inverse RoPE of dq folded in (the backward of rotating q): a thread converts 4 columns of the
// first half of a head and their partners in the second half; token t is at position t % seq.
__global__ void convert_dq_rope_kernel(const float* __restrict__ ws, bf16* __restrict__ dq, long long tokens, int heads, int d,
                                       long long dq_row, const float* __restrict__ cosT, const float* __restrict__ sinT,
                                       int seq) {
  pdl_enter();
  const int half = d / 2, per_head = half / 4;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= tokens * heads * per_head) return;
  const int j = (int)(idx % per_head) * 4;
  const long long th = idx / per_head;
  const int head = (int)(th % heads);
  const long long tok = th / heads;
  const int pos = (int)(tok % seq);
  const float* src = ws + (tok * heads + head) * d + j;
  const float4 a = *reinterpret_cast<const float4*>(src);
  const float4 b = *reinterpret_cast<const float4*>(src + half);
  const float4 c = *reinterpret_cast<const float4*>(cosT + (long long)pos * half + j);
  const float4 sn = *reinterpret_cast<const float4*>(sinT + (long long)pos * half + j);
  uint2 o1, o2;
  o1.x = pack_bf16(a.x * c.x + b.x * sn.x, a.y * c.y + b.y * sn.y);
  o1.y = pack_bf16(a.z * c.z + b.z * sn.z, a.w * c.w + b.w * sn.w);
  o2.x = pack_bf16(b.x * c.x - a.x * sn.x, b.y * c.y - a.y * sn.y);
  o2.y = pack_bf16(b.z * c.z - a.z * sn.z, b.w * c.w - a.w * sn.w);
  bf16* dst = dq + tok * dq_row + (long long)head * d + j;
  *reinterpret_cast<uint2*>(dst) = o1;
  *reinterpret_cast<uint2*>(dst + half) = o2;
}

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// ---------------------------------------------------------------------------------------------------------
// backward main kernel
// ---------------------------------------------------------------------------------------------------------
template <int D>
struct BwdCfg {
  static constexpr int BM = 128;   // query rows per inner step
  static constexpr int BN = 128;   // keys per CTA
  static constexpr int DCH = D / 64;
  static constexpr int TILE_BYTES = 128 * D * 2;         // Q, dO, K, V tiles
  static constexpr int PS_BYTES = BM * BN * 2;           // P and dS tiles
  static constexpr int QSTAGES = (D == 64) ? 3 : 1;      // Q/dO ring: a tile is loaded two steps before its MMAs (d = 64)
  // The dQ tile of a step is staged in shared memory, 128 rows x 32 fp32 columns per buffer, and added to the fp32
  // workspace by one TMA reduce per buffer instead of 8 vector atomics per thread and 32 columns (per-thread atomics
  // were ~half of the step time for d = 128 and saturated L2 for d = 64). Two buffers: d = 64 needs one round, d = 128 two.
  static constexpr bool DQ_TMA = true;
  static constexpr int DQ_BYTES = 2 * BM * 32 * 4;
  static constexpr int SMEM = 2 * TILE_BYTES + QSTAGES * 2 * TILE_BYTES + 2 * PS_BYTES + DQ_BYTES + 1024;
  static constexpr int TMEM_COLS = 512;
  static constexpr bool SHARE_S_DQ = (D == 128);
  static constexpr int S_COL = 0, DP_COL = 128, DV_COL = 256, DK_COL = 256 + D;
  static constexpr int DQ_COL = SHARE_S_DQ ? 0 : 256 + 2 * D;
  static_assert(DQ_COL + D <= 512 && DK_COL + D <= 512, "TMEM budget");
};

struct BwdBars {
  uint64_t kv_full, q_full[3], q_empty[3], s_full, dp_full, pds_ready, dq_full, dq_read, acc_full;
  uint32_t tmem_base;
  int abort_flag;
};

struct BwdParams {
  int B, Sq, Sk, hq, hkv;
  int causal;
  float scale;
  long long dk_row, dv_row;      // token strides (elements) of dk / dv
  int n_segs;
  long long seg_stride;          // elements between the dk (dv) outputs of consecutive segments
  // optional inverse RoPE of the dK output (the backward of rotating k): fp32 [rope_seq, d/2] tables, key i is at
  // position i % rope_seq. Only with one segment and bf16 outputs; nullptr = dK is written as computed.
  const float* cosT;
  const float* sinT;
  int rope_seq;
  unsigned long long* prof;      // optional phase counters, as AttnParams::prof
};

constexpr int BWD_THREADS = 320;   // warps 0-7 compute (two per TMEM lane quarter), warp 8 TMA producer, warp 9 MMA issuer

template <int D, bool OUT_F32, bool PROF>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ KVSegs segs,
                const __grid_constant__ CUtensorMap tm_do, const __grid_constant__ CUtensorMap tm_dq,
                const float* __restrict__ LSE,
                const float* __restrict__ DELTA, float* __restrict__ dq_ws, void* __restrict__ dK_, void* __restrict__ dV_,
                BwdParams p, KernelStatus* status) {
  using Cfg = BwdCfg<D>;
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  __shared__ BwdBars bars;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + Cfg::TILE_BYTES;
  uint8_t* sQ = sV + Cfg::TILE_BYTES;                                 // QSTAGES x (Q tile, dO tile)
  uint8_t* sP = sQ + Cfg::QSTAGES * 2 * Cfg::TILE_BYTES;
  uint8_t* sdS = sP + Cfg::PS_BYTES;
  uint8_t* sDQ = sdS + Cfg::PS_BYTES;                                 // [D/32][128 rows][32 fp32], 128B swizzle (d = 64 only)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bps = (p.Sk + Cfg::BN - 1) / Cfg::BN;         // key blocks per segment
  const int num_kb = bps * p.n_segs;
  const int kbg = (int)(blockIdx.x % num_kb);
  const int seg = kbg / bps;
  const int kb = kbg - seg * bps;
  const bool diag = p.causal && seg == p.n_segs - 1;      // the causal diagonal runs through the last segment only
  const int kv_head = (int)((blockIdx.x / num_kb) % p.hkv);
  const int b = (int)(blockIdx.x / (num_kb * p.hkv));
  const int group = p.hq / p.hkv;
  const int k0 = kb * Cfg::BN;
  const int num_qb = (p.Sq + Cfg::BM - 1) / Cfg::BM;
  const int qb_first = diag ? (k0 / Cfg::BM) : 0;              // first query block that sees key k0
  const int steps_per_head = num_qb - qb_first;
  const int total_steps = steps_per_head > 0 ? steps_per_head * group : 0;

  if (threadIdx.x == 0) {
    mbar_init(&bars.kv_full, 1);
    for (int s = 0; s < 3; ++s) {
      mbar_init(&bars.q_full[s], 1);
      mbar_init(&bars.q_empty[s], 1);
    }
    mbar_init(&bars.s_full, 1);
    mbar_init(&bars.dp_full, 1);
    mbar_init(&bars.pds_ready, 256);
    mbar_init(&bars.dq_full, 1);
    mbar_init(&bars.dq_read, 256);
    mbar_init(&bars.acc_full, 1);
    bars.abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&segs.k[seg]);
    tma_prefetch_desc(&segs.v[seg]);
    tma_prefetch_desc(&tm_do);
  }
  if (warp == 9) {
    tmem_alloc(&bars.tmem_base, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  pdl_wait();                      // barrier init and tensor-memory allocation overlapped the predecessor's tail
  const uint32_t tmem_base = bars.tmem_base;
  volatile int* abort_flag = &bars.abort_flag;

  if (warp == 8) {
    // ------------------------------------------------------------------------------ TMA producer
    if (lane == 0 && total_steps > 0) {
      mbar_expect_tx(&bars.kv_full, 2 * Cfg::TILE_BYTES);
#pragma unroll
      for (int c = 0; c < Cfg::DCH; ++c) {
        tma_load_4d(sK + c * (Cfg::BN * 128), &segs.k[seg], &bars.kv_full, c * 64, kv_head, k0, b);
        tma_load_4d(sV + c * (Cfg::BN * 128), &segs.v[seg], &bars.kv_full, c * 64, kv_head, k0, b);
      }
      for (int it = 0; it < total_steps; ++it) {
        const int st = it % Cfg::QSTAGES;
        const uint32_t ph = (it / Cfg::QSTAGES) & 1;
        const int head = kv_head * group + it / steps_per_head;
        const int qb = qb_first + it % steps_per_head;
        if (!mbar_wait(&bars.q_empty[st], ph ^ 1, abort_flag)) { report_error(status, KID_BWD, 1); break; }
        mbar_expect_tx(&bars.q_full[st], 2 * Cfg::TILE_BYTES);
        uint8_t* q_dst = sQ + st * 2 * Cfg::TILE_BYTES;
        uint8_t* do_dst = q_dst + Cfg::TILE_BYTES;
#pragma unroll
        for (int c = 0; c < Cfg::DCH; ++c) {
          tma_load_4d(q_dst + c * (Cfg::BM * 128), &tm_q, &bars.q_full[st], c * 64, head, qb * Cfg::BM, b);
          tma_load_4d(do_dst + c * (Cfg::BM * 128), &tm_do, &bars.q_full[st], c * 64, head, qb * Cfg::BM, b);
        }
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------------------ MMA issuer
    if (lane == 0 && total_steps > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);   // S, dP: [q, kv], K-major operands
      constexpr uint32_t idesc_kv = make_idesc_bf16(128, D, true, true);      // dV, dK: A = P^T/dS^T, B = dO/Q (both MN-major)
      constexpr uint32_t idesc_dq = make_idesc_bf16(128, D, false, true);     // dQ: A = dS (K-major), B = K (MN-major)
      bool ok = mbar_wait(&bars.kv_full, 0, abort_flag);
      if (!ok) report_error(status, KID_BWD, 2);
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV), p_addr = smem_u32(sP), ds_addr = smem_u32(sdS);
      // Base descriptors, built once: one thread issues ~40 MMAs per step and is on the critical path of every hand-off,
      // so the per-MMA work is kept to two integer adds. "km" = K-major view (LBO 16), "mn" = MN-major view (LBO = tile).
      const uint64_t k_km = make_smem_desc_sw128(k_addr, 16, 1024), k_mn = make_smem_desc_sw128(k_addr, 128 * 128, 1024);
      const uint64_t v_km = make_smem_desc_sw128(v_addr, 16, 1024);
      const uint64_t p_mn = make_smem_desc_sw128(p_addr, 128 * 128, 1024);
      const uint64_t ds_mn = make_smem_desc_sw128(ds_addr, 128 * 128, 1024), ds_km = make_smem_desc_sw128(ds_addr, 16, 1024);
      // S = Q K^T and dP = dO V^T of step `it`
      auto issue_s_dp = [&](int it) -> bool {
        const int st = it % Cfg::QSTAGES;
        const uint32_t q_addr = smem_u32(sQ + st * 2 * Cfg::TILE_BYTES);
        const uint64_t q_km = make_smem_desc_sw128(q_addr, 16, 1024);
        const uint64_t do_km = smem_desc_advance(q_km, Cfg::TILE_BYTES);
        if (!mbar_wait(&bars.q_full[st], (it / Cfg::QSTAGES) & 1, abort_flag)) { report_error(status, KID_BWD, 3); return false; }
        if (Cfg::SHARE_S_DQ && it > 0) {   // S overwrites the columns dQ of the previous step was read from
          if (!mbar_wait(&bars.dq_read, (it - 1) & 1, abort_flag)) { report_error(status, KID_BWD, 4); return false; }
        }
        tcgen05_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * (128 * 128) + (kk & 3) * 32;
          umma_bf16(tmem_base + Cfg::S_COL, smem_desc_advance(q_km, off), smem_desc_advance(k_km, off), idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&bars.s_full);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * (128 * 128) + (kk & 3) * 32;
          umma_bf16(tmem_base + Cfg::DP_COL, smem_desc_advance(do_km, off), smem_desc_advance(v_km, off), idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&bars.dp_full);
        return true;
      };
      for (int it = 0; it < total_steps && ok; ++it) {
        const int st = it % Cfg::QSTAGES;
        const uint64_t q_mn = make_smem_desc_sw128(smem_u32(sQ + st * 2 * Cfg::TILE_BYTES), 128 * 128, 1024);
        const uint64_t do_mn = smem_desc_advance(q_mn, Cfg::TILE_BYTES);
        if (!issue_s_dp(it)) break;
        if (!mbar_wait(&bars.pds_ready, it & 1, abort_flag)) { report_error(status, KID_BWD, 5); break; }
        if (!Cfg::SHARE_S_DQ && it > 0) {  // separate dQ columns: only the previous dQ must have been read
          if (!mbar_wait(&bars.dq_read, (it - 1) & 1, abort_flag)) { report_error(status, KID_BWD, 6); break; }
        }
        tcgen05_fence_after();
        // dQ = dS K : M = 128 query rows, N = D, reduction over the 128 keys. Issued first: the compute threads drain
        // dQ while the (three times longer) dV/dK MMAs below still run.
#pragma unroll
        for (int kk = 0; kk < 128 / 16; ++kk)
          umma_bf16(tmem_base + Cfg::DQ_COL, smem_desc_advance(ds_km, (kk >> 2) * (128 * 128) + (kk & 3) * 32),
                    smem_desc_advance(k_mn, kk * 2048), idesc_dq, kk > 0 ? 1u : 0u);
        umma_commit(&bars.dq_full);
        // dV += P^T dO, dK += dS^T Q : M = 128 keys, N = D, reduction over the 128 query rows. The next step's P / dS
        // are only written after s_full of that step, whose commit also covers these MMAs.
#pragma unroll
        for (int kk = 0; kk < 128 / 16; ++kk) {
          // A: P / dS stored [q rows][kv], kv contiguous -> MN-major with M = kv: two 64-key chunks (LBO), 8-row groups (SBO)
          // B: dO / Q stored [q rows][d], d contiguous -> MN-major with N = d
          umma_bf16(tmem_base + Cfg::DV_COL, smem_desc_advance(p_mn, kk * 2048), smem_desc_advance(do_mn, kk * 2048), idesc_kv,
                    (it > 0 || kk > 0) ? 1u : 0u);
          umma_bf16(tmem_base + Cfg::DK_COL, smem_desc_advance(ds_mn, kk * 2048), smem_desc_advance(q_mn, kk * 2048), idesc_kv,
                    (it > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&bars.q_empty[st]);
      }
      if (ok) umma_commit(&bars.acc_full);
    }
  } else {
    // ------------------------------------------------------------------------------ compute threads (warps 0..7)
    // Thread pair (t, t + 128) shares query row t (TMEM lane t): `half` 0 owns score columns 0..63, dQ columns
    // 0..D/2-1 and the dV output, `half` 1 the rest and dK. Nothing has to be exchanged between the two.
    const int t = threadIdx.x & 127;
    const int half = threadIdx.x >> 7;
    const uint32_t t_lane = tmem_base + (uint32_t((warp & 3) * 32) << 16);
    const float sl2 = p.scale * LOG2E;
    bool ok = total_steps > 0;
    const bool prof_on = PROF && p.prof != nullptr && threadIdx.x == 0;
    long long pacc[4] = {0, 0, 0, 0};
    const long long pstart = prof_clock(prof_on);
    for (int it = 0; it < total_steps; ++it) {
      const long long pt0 = prof_clock(prof_on);
      const int head = kv_head * group + it / steps_per_head;
      const int qb = qb_first + it % steps_per_head;
      const int row = qb * Cfg::BM + t;
      const bool row_ok = row < p.Sq;
      const long long stat_idx = ((long long)b * p.hq + head) * p.Sq + (row_ok ? row : 0);
      const float lse2 = row_ok ? LSE[stat_idx] * LOG2E : 0.f;
      const float dlt = row_ok ? DELTA[stat_idx] : 0.f;
      const bool need_mask = (diag && k0 + Cfg::BN - 1 > qb * Cfg::BM) || (k0 + Cfg::BN > p.Sk) || !row_ok;
      if (!mbar_wait(&bars.s_full, it & 1, abort_flag)) { if (lane == 0) report_error(status, KID_BWD, 7); ok = false; break; }
      if (!mbar_wait(&bars.dp_full, it & 1, abort_flag)) { if (lane == 0) report_error(status, KID_BWD, 8); ok = false; break; }
      tcgen05_fence_after();
      const long long pt1 = prof_clock(prof_on);
      uint32_t rs[64], rd[64];                       // this thread's 64 score / dP columns, one batched TMEM read
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        tmem_ld_32x32b_x32_at(t_lane + Cfg::S_COL + (half * 2 + cc) * 32, rs, cc * 32);
        tmem_ld_32x32b_x32_at(t_lane + Cfg::DP_COL + (half * 2 + cc) * 32, rd, cc * 32);
      }
      tmem_ld_wait();
      const float dlt_s = dlt * p.scale;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = half * 2 + cc;
        uint32_t pp[16], dd[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float p0 = fast_exp2(__uint_as_float(rs[cc * 32 + e]) * sl2 - lse2);
          float p1 = fast_exp2(__uint_as_float(rs[cc * 32 + e + 1]) * sl2 - lse2);
          if (need_mask) {
            const int col = k0 + c * 32 + e;
            if (!row_ok || (diag && col > row) || col >= p.Sk) p0 = 0.f;
            if (!row_ok || (diag && col + 1 > row) || col + 1 >= p.Sk) p1 = 0.f;
          }
          const float d0 = p0 * (__uint_as_float(rd[cc * 32 + e]) * p.scale - dlt_s);
          const float d1 = p1 * (__uint_as_float(rd[cc * 32 + e + 1]) * p.scale - dlt_s);
          pp[e >> 1] = pack_bf16(p0, p1);
          dd[e >> 1] = pack_bf16(d0, d1);
        }
        const uint32_t chunk_off = ((c * 32) >> 6) * (128 * 128);
        const int u0 = ((c * 32) & 63) >> 3;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const uint32_t off = chunk_off + sw128_offset(t, u0 + u);
          *reinterpret_cast<uint4*>(sP + off) = make_uint4(pp[4 * u], pp[4 * u + 1], pp[4 * u + 2], pp[4 * u + 3]);
          *reinterpret_cast<uint4*>(sdS + off) = make_uint4(dd[4 * u], dd[4 * u + 1], dd[4 * u + 2], dd[4 * u + 3]);
        }
      }
      tcgen05_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(&bars.pds_ready);
      const long long pt2 = prof_clock(prof_on);
      // dQ tile of this step -> fp32 workspace
      if (!mbar_wait(&bars.dq_full, it & 1, abort_flag)) { if (lane == 0) report_error(status, KID_BWD, 9); ok = false; break; }
      tcgen05_fence_after();
      const long long pt3 = prof_clock(prof_on);
      if (Cfg::DQ_TMA) {
        // round r: `half` h stages dQ columns [32 (h R + r), +32) of its row (R = D / 64 rounds); thread 0 hands both
        // 128 x 32 buffers to TMA
#pragma unroll 1
        for (int r_ = 0; r_ < D / 64; ++r_) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_lane + Cfg::DQ_COL + (half * (D / 64) + r_) * 32, r);
          tmem_ld_wait();
          if (threadIdx.x == 0) tma_store_wait_read<0>();   // the previous reduce has finished reading the staging buffers
          asm volatile("bar.sync 1, 256;" ::: "memory");
#pragma unroll
          for (int u = 0; u < 8; ++u)
            *reinterpret_cast<uint4*>(sDQ + half * (128 * 128) + sw128_offset(t, u)) =
                make_uint4(r[4 * u], r[4 * u + 1], r[4 * u + 2], r[4 * u + 3]);
          fence_proxy_async_smem();
          asm volatile("bar.sync 1, 256;" ::: "memory");
          if (threadIdx.x == 0) {
#pragma unroll
            for (int h = 0; h < 2; ++h)
              tma_reduce_add_4d(&tm_dq, sDQ + h * (128 * 128), (h * (D / 64) + r_) * 32, head, qb * Cfg::BM, b);
            tma_store_commit();
          }
        }
      } else {
        float* dq_row = dq_ws + (((long long)b * p.Sq + (row_ok ? row : 0)) * p.hq + head) * D + half * (D / 2);
#pragma unroll 1
        for (int c = 0; c < D / 64; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_lane + Cfg::DQ_COL + half * (D / 2) + c * 32, r);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int e = 0; e < 32; e += 4)
              red_add_v4(dq_row + c * 32 + e, __uint_as_float(r[e]), __uint_as_float(r[e + 1]), __uint_as_float(r[e + 2]),
                         __uint_as_float(r[e + 3]));
          }
        }
      }
      tcgen05_fence_before();
      mbar_arrive(&bars.dq_read);
      if (prof_on) {
        const long long pt4 = clock64();
        pacc[0] += pt1 - pt0; pacc[1] += pt2 - pt1; pacc[2] += pt3 - pt2; pacc[3] += pt4 - pt3;
      }
    }
    if (prof_on) {
      for (int i = 0; i < 4; ++i) atomicAdd(&p.prof[i], (unsigned long long)pacc[i]);
      atomicAdd(&p.prof[4], (unsigned long long)total_steps);
      atomicAdd(&p.prof[5], (unsigned long long)(clock64() - pstart));
      atomicAdd(&p.prof[6], 1ull);
    }
    if (Cfg::DQ_TMA && threadIdx.x == 0) tma_store_wait<0>();
    // dK, dV of this key block (thread t <-> key k0 + t); fp32 when they are partials of a multi-rank reduction
    const int key = k0 + t;
    const long long seg_off = (long long)seg * p.seg_stride;
    if (total_steps == 0) {
      if (key < p.Sk) {
        {
          const int which = half;                  // half 0 writes dV, half 1 writes dK
          const long long rs_ = which == 0 ? p.dv_row : p.dk_row;
          const long long off = seg_off + ((long long)b * p.Sk + key) * rs_ + (long long)kv_head * D;
          if (OUT_F32) {
            float* orow = reinterpret_cast<float*>(which == 0 ? dV_ : dK_) + off;
            for (int u = 0; u < D / 4; ++u) reinterpret_cast<float4*>(orow)[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          } else {
            bf16* orow = reinterpret_cast<bf16*>(which == 0 ? dV_ : dK_) + off;
            for (int u = 0; u < D / 8; ++u) reinterpret_cast<uint4*>(orow)[u] = make_uint4(0, 0, 0, 0);
          }
        }
      }
    } else if (ok && mbar_wait(&bars.acc_full, 0, abort_flag)) {
      tcgen05_fence_after();
      if (!OUT_F32 && half == 1 && p.cosT != nullptr) {
        // dK with the inverse rotation: the whole row (D columns) in registers, pairs j <-> j + D/2
        uint32_t r[D];
#pragma unroll
        for (int c = 0; c < D / 32; ++c) tmem_ld_32x32b_x32_at(t_lane + Cfg::DK_COL + c * 32, r, c * 32);
        tmem_ld_wait();
        if (key < p.Sk) {
          const int pos = key % p.rope_seq;
          const float* cos_row = p.cosT + (long long)pos * (D / 2);
          const float* sin_row = p.sinT + (long long)pos * (D / 2);
#pragma unroll
          for (int j = 0; j < D / 2; j += 4) {
            const float4 cs = __ldg(reinterpret_cast<const float4*>(cos_row + j));
            const float4 sn = __ldg(reinterpret_cast<const float4*>(sin_row + j));
            const float csv[4] = {cs.x, cs.y, cs.z, cs.w}, snv[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float a = __uint_as_float(r[j + i]), b = __uint_as_float(r[j + i + D / 2]);
              r[j + i] = __float_as_uint(a * csv[i] + b * snv[i]);
              r[j + i + D / 2] = __float_as_uint(b * csv[i] - a * snv[i]);
            }
          }
          bf16* orow = reinterpret_cast<bf16*>(dK_) + seg_off + ((long long)b * p.Sk + key) * p.dk_row + (long long)kv_head * D;
#pragma unroll
          for (int u = 0; u < D / 8; ++u)
            reinterpret_cast<uint4*>(orow)[u] =
                make_uint4(pack_bf16(__uint_as_float(r[8 * u]), __uint_as_float(r[8 * u + 1])),
                           pack_bf16(__uint_as_float(r[8 * u + 2]), __uint_as_float(r[8 * u + 3])),
                           pack_bf16(__uint_as_float(r[8 * u + 4]), __uint_as_float(r[8 * u + 5])),
                           pack_bf16(__uint_as_float(r[8 * u + 6]), __uint_as_float(r[8 * u + 7])));
        }
      } else {
        const int which = half;                    // half 0 writes dV, half 1 writes dK
        const long long rs_ = which == 0 ? p.dv_row : p.dk_row;
        const int col_base = which == 0 ? Cfg::DV_COL : Cfg::DK_COL;
        const long long off = seg_off + ((long long)b * p.Sk + (key < p.Sk ? key : 0)) * rs_ + (long long)kv_head * D;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_lane + col_base + c * 32, r);
          tmem_ld_wait();
          if (key < p.Sk) {
            if (OUT_F32) {
              float* orow = reinterpret_cast<float*>(which == 0 ? dV_ : dK_) + off + c * 32;
#pragma unroll
              for (int u = 0; u < 8; ++u)
                reinterpret_cast<float4*>(orow)[u] = make_float4(__uint_as_float(r[4 * u]), __uint_as_float(r[4 * u + 1]),
                                                                 __uint_as_float(r[4 * u + 2]), __uint_as_float(r[4 * u + 3]));
            } else {
              bf16* orow = reinterpret_cast<bf16*>(which == 0 ? dV_ : dK_) + off + c * 32;
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                uint4 v = make_uint4(pack_bf16(__uint_as_float(r[8 * u]), __uint_as_float(r[8 * u + 1])),
                                     pack_bf16(__uint_as_float(r[8 * u + 2]), __uint_as_float(r[8 * u + 3])),
                                     pack_bf16(__uint_as_float(r[8 * u + 4]), __uint_as_float(r[8 * u + 5])),
                                     pack_bf16(__uint_as_float(r[8 * u + 6]), __uint_as_float(r[8 * u + 7])));
                reinterpret_cast<uint4*>(orow)[u] = v;
              }
            }
          }
        }
      }
    } else if (ok && lane == 0) {
      report_error(status, KID_BWD, 10);
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 9) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------
// tensor map over x[B, S, h, d] with token stride `row` (elements): dims {d, h, S, B}, box {64, 1, rows, 1}
static int make_attn_map(CUtensorMap* m, const void* base, int B, int S, int h, int d, long long row, int box_rows) {
  uint64_t dims[4] = {(uint64_t)d, (uint64_t)h, (uint64_t)S, (uint64_t)B};
  uint64_t strides[3] = {(uint64_t)d, (uint64_t)row, (uint64_t)row * (uint64_t)S};
  uint32_t box[4] = {64, 1, (uint32_t)box_rows, 1};
  return make_bf16_map(m, base, 4, dims, strides, box);
}

template <int D, int BN, bool PROF = false>
static int launch_fwd(const CUtensorMap& mq, const KVSegs& segs, void* o, float* lse, const AttnParams& p,
                      KernelStatus* st, cudaStream_t stream) {
  if (!PROF && p.prof != nullptr) return launch_fwd<D, BN, true>(mq, segs, o, lse, p, st, stream);
  auto kern = attn_fwd_kernel<D, BN, PROF>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdCfg<D, BN>::SMEM) != cudaSuccess) return -3;
    // two CTAs per SM need the largest shared-memory carve-out
    cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    configured = true;
  }
  const int num_qb = (p.Sq + 127) / 128;
  const long long grid = (long long)num_qb * p.hq * p.B;
  launch_pdl(kern, dim3((unsigned)grid), dim3(192), FwdCfg<D, BN>::SMEM, stream, mq, segs, (bf16*)o, lse, p, st);
  pt_count_launches(1);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

template <int D, bool OUT_F32, bool PROF = false>
static int launch_bwd(const CUtensorMap& mq, const KVSegs& segs, const CUtensorMap& mdo, const CUtensorMap& mdq, const float* lse,
                      const float* delta, float* dq_ws, void* dk, void* dv, const BwdParams& p, KernelStatus* st,
                      cudaStream_t stream) {
  if (!PROF && p.prof != nullptr)
    return launch_bwd<D, OUT_F32, true>(mq, segs, mdo, mdq, lse, delta, dq_ws, dk, dv, p, st, stream);
  auto kern = attn_bwd_kernel<D, OUT_F32, PROF>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdCfg<D>::SMEM) != cudaSuccess) return -3;
    cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    configured = true;
  }
  const int num_kb = ((p.Sk + 127) / 128) * p.n_segs;
  const long long grid = (long long)num_kb * p.hkv * p.B;
  launch_pdl(kern, dim3((unsigned)grid), dim3(BWD_THREADS), BwdCfg<D>::SMEM, stream, mq, segs, mdo, mdq, lse, delta, dq_ws, dk, dv, p, st);
  pt_count_launches(1);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace attn
}  // namespace pt

// q [B,Sq,hq,d] bf16 with token stride q_row; K/V in `n_segs` segments: k_ptrs[i]/v_ptrs[i] are [B,Sk,hkv,d] bf16 with
// token strides k_row/v_row (elements, multiples of 8) and may be peer-mapped pointers into other GPUs' memory.
// `causal` masks inside the last segment only. o [B,Sq,hq,d] bf16 contiguous; lse [B,hq,Sq] fp32 (natural log).
extern "C" int pt_attention_fwd_segs(const void* q, const void* const* k_ptrs, const void* const* v_ptrs, int n_segs,
                                     void* o, float* lse, int B, int Sq, int Sk, int hq, int hkv, int d, long long q_row,
                                     long long k_row, long long v_row, int causal, float scale, cudaStream_t st) {
  using namespace pt;
  using namespace pt::attn;
  if (B <= 0 || Sq <= 0 || Sk <= 0) return 0;
  if ((d != 64 && d != 128) || hq % hkv || (q_row % 8) || (k_row % 8) || (v_row % 8) || n_segs < 1 || n_segs > MAX_SEGS)
    return -10;
  CUtensorMap mq;
  KVSegs segs;
  const int bn = d == 64 ? 128 : 64;
  int rc;
  if ((rc = make_attn_map(&mq, q, B, Sq, hq, d, q_row, 128))) return rc;
  for (int i = 0; i < n_segs; ++i) {
    if ((rc = make_attn_map(&segs.k[i], k_ptrs[i], B, Sk, hkv, d, k_row, bn))) return rc;
    if ((rc = make_attn_map(&segs.v[i], v_ptrs[i], B, Sk, hkv, d, v_row, bn))) return rc;
  }
  for (int i = n_segs; i < MAX_SEGS; ++i) { segs.k[i] = segs.k[0]; segs.v[i] = segs.v[0]; }
  AttnParams p{B, Sq, Sk, hq, hkv, causal, scale, n_segs, g_attn_prof};
  if (d == 64) return launch_fwd<64, 128>(mq, segs, o, lse, p, status_word_attn(), st);
  return launch_fwd<128, 64>(mq, segs, o, lse, p, status_word_attn(), st);
}

extern "C" int pt_attention_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Sq, int Sk,
                                int hq, int hkv, int d, long long q_row, long long k_row, long long v_row, int causal,
                                float scale, cudaStream_t st) {
  return pt_attention_fwd_segs(q, &k, &v, 1, o, lse, B, Sq, Sk, hq, hkv, d, q_row, k_row, v_row, causal, scale, st);
}

// Backward over `n_segs` K/V segments (see pt_attention_fwd_segs). dout, o [B,Sq,hq,d] bf16 contiguous; lse [B,hq,Sq];
// delta_in optional (else computed into delta_ws [B,hq,Sq]); dq_ws fp32 [B,Sq,hq,d] zero-initialised scratch; dq bf16 with
// token stride dq_row. dk/dv: outputs of segment i start i*seg_stride elements after dk/dv, token strides dk_row/dv_row,
// bf16 or (out_f32) fp32 -- fp32 is used when they are partial sums that another rank reduces.
static int attention_bwd_impl(const void* dout, const void* q, const void* const* k_ptrs, const void* const* v_ptrs,
                                     int n_segs, const void* o, const float* lse, const float* delta_in, float* delta_ws,
                                     float* dq_ws, void* dq, void* dk, void* dv, int out_f32, long long seg_stride, int B,
                                     int Sq, int Sk, int hq, int hkv, int d, long long q_row, long long k_row,
                                     long long v_row, long long dq_row, long long dk_row, long long dv_row, int causal,
                                     float scale, cudaStream_t st, const float* cosT, const float* sinT, int rope_seq) {
  using namespace pt;
  using namespace pt::attn;
  if (B <= 0 || Sq <= 0 || Sk <= 0) return 0;
  if ((d != 64 && d != 128) || hq % hkv || (q_row % 8) || (k_row % 8) || (v_row % 8) || (dq_row % 4) || (dk_row % 8) ||
      (dv_row % 8) || n_segs < 1 || n_segs > MAX_SEGS)
    return -10;
  const float* delta = delta_in;
  if (delta == nullptr) {
    const long long threads = (long long)B * Sq * hq * (d / 8);
    const unsigned blocks = (unsigned)((threads + 255) / 256);
    if (d == 64) launch_pdl(delta_kernel<64>, dim3(blocks), dim3(256), 0, st, (const bf16*)dout, (const bf16*)o, delta_ws, B, Sq, hq);
    else launch_pdl(delta_kernel<128>, dim3(blocks), dim3(256), 0, st, (const bf16*)dout, (const bf16*)o, delta_ws, B, Sq, hq);
    pt_count_launches(1);
    delta = delta_ws;
  }
  CUtensorMap mq, mdo, mdq;
  KVSegs segs;
  int rc;
  if ((rc = make_attn_map(&mq, q, B, Sq, hq, d, q_row, 128))) return rc;
  if ((rc = make_attn_map(&mdo, dout, B, Sq, hq, d, (long long)hq * d, 128))) return rc;
  {
    // fp32 dQ workspace [B, Sq, hq, d]: 32-column x 128-row boxes for the TMA reduce-add (used by the d = 64 kernel)
    uint64_t dims[4] = {(uint64_t)d, (uint64_t)hq, (uint64_t)Sq, (uint64_t)B};
    uint64_t strides[3] = {(uint64_t)d, (uint64_t)hq * d, (uint64_t)hq * d * (uint64_t)Sq};
    uint32_t box[4] = {32, 1, 128, 1};
    if ((rc = make_f32_map(&mdq, dq_ws, 4, dims, strides, box))) return rc;
  }
  for (int i = 0; i < n_segs; ++i) {
    if ((rc = make_attn_map(&segs.k[i], k_ptrs[i], B, Sk, hkv, d, k_row, 128))) return rc;
    if ((rc = make_attn_map(&segs.v[i], v_ptrs[i], B, Sk, hkv, d, v_row, 128))) return rc;
  }
  for (int i = n_segs; i < MAX_SEGS; ++i) { segs.k[i] = segs.k[0]; segs.v[i] = segs.v[0]; }
  if (cosT != nullptr && (n_segs != 1 || out_f32 || sinT == nullptr || rope_seq <= 0 || (reinterpret_cast<uintptr_t>(cosT) & 15) ||
                          (reinterpret_cast<uintptr_t>(sinT) & 15)))
    return -12;
  BwdParams p{B, Sq, Sk, hq, hkv, causal, scale, dk_row, dv_row, n_segs, seg_stride, cosT, sinT, rope_seq, g_attn_prof};
  KernelStatus* sw = status_word_attn();
  if (d == 64) rc = out_f32 ? launch_bwd<64, true>(mq, segs, mdo, mdq, lse, delta, dq_ws, dk, dv, p, sw, st)
                            : launch_bwd<64, false>(mq, segs, mdo, mdq, lse, delta, dq_ws, dk, dv, p, sw, st);
  else rc = out_f32 ? launch_bwd<128, true>(mq, segs, mdo, mdq, lse, delta, dq_ws, dk, dv, p, sw, st)
                    : launch_bwd<128, false>(mq, segs, mdo, mdq, lse, delta, dq_ws, dk, dv, p, sw, st);
  if (rc) return rc;
  if (dq != nullptr) {
    const long long n = (long long)B * Sq * hq * d;
    if (cosT != nullptr)
      launch_pdl(convert_dq_rope_kernel, dim3((unsigned)((n / 8 + 255) / 256)), dim3(256), 0, st, dq_ws, (bf16*)dq, (long long)B * Sq,
                 hq, d, dq_row, cosT, sinT, rope_seq);
    else
      launch_pdl(convert_dq_kernel, dim3((unsigned)((n / 4 + 255) / 256)), dim3(256), 0, st, dq_ws, (bf16*)dq, (long long)B * Sq,
                 hq * d, dq_row);
    pt_count_launches(1);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int pt_attention_bwd_segs(const void* dout, const void* q, const void* const* k_ptrs, const void* const* v_ptrs,
                                     int n_segs, const void* o, const float* lse, const float* delta_in, float* delta_ws,
                                     float* dq_ws, void* dq, void* dk, void* dv, int out_f32, long long seg_stride, int B, int Sq,
                                     int Sk, int hq, int hkv, int d, long long q_row, long long k_row, long long v_row,
                                     long long dq_row, long long dk_row, long long dv_row, int causal, float scale,
                                     cudaStream_t st) {
  return attention_bwd_impl(dout, q, k_ptrs, v_ptrs, n_segs, o, lse, delta_in, delta_ws, dq_ws, dq, dk, dv, out_f32, seg_stride, B,
                            Sq, Sk, hq, hkv, d, q_row, k_row, v_row, dq_row, dk_row, dv_row, causal, scale, st, nullptr, nullptr, 0);
}

// pt_attention_bwd that also undoes RoPE on its dq and dk outputs (the backward of rotating q and k before attention):
// cosT/sinT fp32 [rope_seq, d/2], 16-byte aligned; query / key i sits at position i % rope_seq.
extern "C" int pt_attention_bwd_rope(const void* dout, const void* q, const void* k, const void* v, const void* o,
                                     const float* lse, const float* delta_in, float* delta_ws, float* dq_ws, void* dq,
                                     void* dk, void* dv, int B, int Sq, int Sk, int hq, int hkv, int d, long long q_row,
                                     long long k_row, long long v_row, long long dq_row, long long dk_row, long long dv_row,
                                     int causal, float scale, const float* cosT, const float* sinT, int rope_seq,
                                     cudaStream_t st) {
  return attention_bwd_impl(dout, q, &k, &v, 1, o, lse, delta_in, delta_ws, dq_ws, dq, dk, dv, 0, 0, B, Sq, Sk, hq, hkv, d, q_row,
                            k_row, v_row, dq_row, dk_row, dv_row, causal, scale, st, cosT, sinT, rope_seq);
}

extern "C" int pt_attention_bwd(const void* dout, const void* q, const void* k, const void* v, const void* o,
                                const float* lse, const float* delta_in, float* delta_ws, float* dq_ws, void* dq,
                                void* dk, void* dv, int B, int Sq, int Sk, int hq, int hkv, int d, long long q_row,
                                long long k_row, long long v_row, long long dq_row, long long dk_row, long long dv_row,
                                int causal, float scale, cudaStream_t st) {
  return pt_attention_bwd_segs(dout, q, &k, &v, 1, o, lse, delta_in, delta_ws, dq_ws, dq, dk, dv, 0, 0, B, Sq, Sk, hq, hkv,
                               d, q_row, k_row, v_row, dq_row, dk_row, dv_row, causal, scale, st);
}

// Phase profiling of the attention kernels: `counters` is a device buffer of 16 uint64 that subsequent forward / backward
// launches add their phase cycle counts to (layout next to AttnParams); nullptr switches it off again.
extern "C" void pt_attention_set_profile(unsigned long long* counters) { pt::attn::g_attn_prof = counters; }

// Peer-memory collectives over NVLink / NVSwitch for buffers that live in symmetric memory (the same
// allocation mapped at every rank of a group, peers' base pointers known to every rank).
//
// They replace the NCCL all-reduces of the reference: the bucketed data-parallel gradient average
// (picotron/data_parallel/bucket.py:25-31: `grad /= n; all_reduce`), the tensor-parallel activation and
// gradient all-reduces (picotron/tensor_parallel/tp_communications.py:19-49).
//
// all-reduce, in place, two-shot inside ONE kernel:
//   1. start barrier   block b of every rank tells block b of every peer "my buffer holds its contribution"
//   2. reduce-scatter  rank r sums slice r of all ranks in fp32 (peer loads, or ONE multimem.ld_reduce
//                      through the switch when the buffer has a multicast mapping), applies `scale`
//                      (1/n for gradient averaging: the reference's separate division pass is fused here)
//   3. all-gather      the result is stored into slice r of every rank (peer stores, or ONE multimem.st)
//   4. done barrier    block b waits until every peer's block b finished writing into this rank
// Flags are monotonically increasing epochs in symmetric memory (no reset, a stale flag is recognisable);
// every wait has a deadline and records a status code instead of spinning forever.
//
// The epoch of a call is not a host argument: every workspace keeps its call counter in device memory (two control
// words in its own flag region). Each block reads `counter + 1` when it starts, and the last block to finish stores the
// new value, so the same launch can be replayed from a CUDA graph any number of times and stays in step with the peers
// as long as all ranks run the same sequence of collectives on the workspace (launches on one workspace must be
// ordered on one stream). The wait limit is a launch argument taken from a process-wide setting (pt_set_wait_limit_ns).
#include "common.cuh"

extern "C" void pt_count_launches(int n);
extern "C" void* pt_status_word();

namespace pt {
namespace comm {

constexpr int MAX_RANKS = 8;
constexpr int MAX_BLOCKS = 128;
constexpr unsigned KID_AR = 5;
constexpr unsigned long long kDefaultWaitNs = 4000000000ULL;   // 4 s
// control words of a workspace: uint32 index into its flag region (behind the 8 KiB of barrier flags)
constexpr size_t CTRL_WORDS_OFFSET = 8192 / 4;

struct Peers {
  void* buf[MAX_RANKS];          // base of the data region at every rank (peer-mapped)
  unsigned int* flags[MAX_RANKS];  // flag region at every rank: [2][MAX_RANKS][MAX_BLOCKS] uint32
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

// Epoch of this launch: one more than the workspace's call counter (same value in every block: the counter is only
// advanced by the last block that FINISHES, see end_call).
__device__ __forceinline__ unsigned int begin_call(unsigned int* ctrl) {
  __shared__ unsigned int epoch_s;
  if (threadIdx.x == 0) epoch_s = *reinterpret_cast<volatile unsigned int*>(ctrl) + 1u;
  __syncthreads();
  return epoch_s;
}
// Called by every block on every path out of the kernel (also after a timed-out wait, so that later launches still agree
// with each other on this rank).
__device__ __forceinline__ void end_call(unsigned int* ctrl, unsigned int epoch) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int arrived = atomicAdd(ctrl + 1, 1u);
    if (arrived == gridDim.x - 1) {
      ctrl[1] = 0u;
      __threadfence();
      *reinterpret_cast<volatile unsigned int*>(ctrl) = epoch;
    }
  }
}

// Block-level barrier across ranks. `phase` 0 = start, 1 = done. Returns false on timeout.
__device__ __forceinline__ bool cross_rank_barrier(const Peers& peers, int rank, int world, int phase, unsigned int epoch,
                                                   KernelStatus* status, unsigned long long wait_ns) {
  __shared__ int ok_flag;
  __syncthreads();
  if (threadIdx.x == 0) ok_flag = 1;
  __syncthreads();
  if (threadIdx.x < world) {
    const int q = threadIdx.x;
    __threadfence_system();
    // tell rank q's block b that rank `rank` reached this phase
    st_release_sys(peers.flags[q] + ((size_t)phase * MAX_RANKS + rank) * MAX_BLOCKS + blockIdx.x, epoch);
    // wait for rank q's block b
    const unsigned int* mine = peers.flags[rank] + ((size_t)phase * MAX_RANKS + q) * MAX_BLOCKS + blockIdx.x;
    const unsigned long long t0 = globaltimer_ns();
    unsigned spins = 0;
    while ((int)(ld_acquire_sys(mine) - epoch) < 0) {
      if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > wait_ns) {
        ok_flag = 0;
        report_error(status, KID_AR, 1 + phase);
        break;
      }
    }
  }
  __syncthreads();
  return ok_flag != 0;
}

__device__ __forceinline__ float4 ld_f4(const float* p) { return *reinterpret_cast<const float4*>(p); }

template <bool MULTIMEM>
__global__ void __launch_bounds__(512)
allreduce_f32_kernel(Peers peers, float* mc_base, long long offset_elems, long long n, float scale, int rank, int world,
                     unsigned long long wait_ns, KernelStatus* status) {
  unsigned int* ctrl = peers.flags[rank] + CTRL_WORDS_OFFSET;
  const unsigned int epoch = begin_call(ctrl);
  if (!cross_rank_barrier(peers, rank, world, 0, epoch, status, wait_ns)) {
    end_call(ctrl, epoch);
    return;
  }
  // slice of this rank, in float4 units
  const long long n4 = n / 4;
  const long long per = (n4 + world - 1) / world;
  const long long lo = min(n4, per * rank), hi = min(n4, per * (rank + 1));
  // eight independent 16-byte transactions per thread in flight (NVLink latency is microseconds)
  constexpr int UNROLL = 8;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = lo + (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < hi; i0 += stride * UNROLL) {
    float4 acc[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long i = i0 + u * stride;
      acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i < hi) {
        if (MULTIMEM) {
          float* a = mc_base + offset_elems + i * 4;
          asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                       : "=f"(acc[u].x), "=f"(acc[u].y), "=f"(acc[u].z), "=f"(acc[u].w) : "l"(a) : "memory");
        } else {
          for (int q = 0; q < world; ++q) {
            const float4 v = ld_f4(reinterpret_cast<const float*>(peers.buf[q]) + offset_elems + i * 4);
            acc[u].x += v.x; acc[u].y += v.y; acc[u].z += v.z; acc[u].w += v.w;
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long i = i0 + u * stride;
      if (i < hi) {
        const float4 r = make_float4(acc[u].x * scale, acc[u].y * scale, acc[u].z * scale, acc[u].w * scale);
        if (MULTIMEM) {
          float* a = mc_base + offset_elems + i * 4;
          asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(a), "f"(r.x), "f"(r.y),
                       "f"(r.z), "f"(r.w) : "memory");
        } else {
          for (int q = 0; q < world; ++q)
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(peers.buf[q]) + offset_elems + i * 4) = r;
        }
      }
    }
  }
  // tail (n not a multiple of 4): rank 0, plain loads/stores
  if (rank == 0 && blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const long long i = n4 * 4 + threadIdx.x;
    float acc = 0.f;
    for (int q = 0; q < world; ++q) acc += reinterpret_cast<const float*>(peers.buf[q])[offset_elems + i];
    acc *= scale;
    for (int q = 0; q < world; ++q) reinterpret_cast<float*>(peers.buf[q])[offset_elems + i] = acc;
  }
  cross_rank_barrier(peers, rank, world, 1, epoch, status, wait_ns);
  end_call(ctrl, epoch);
}

template <bool MULTIMEM>
__global__ void __launch_bounds__(512)
allreduce_bf16_kernel(Peers peers, __nv_bfloat16* mc_base, long long offset_elems, long long n, int rank, int world,
                      unsigned long long wait_ns, KernelStatus* status) {
  unsigned int* ctrl = peers.flags[rank] + CTRL_WORDS_OFFSET;
  const unsigned int epoch = begin_call(ctrl);
  if (!cross_rank_barrier(peers, rank, world, 0, epoch, status, wait_ns)) {
    end_call(ctrl, epoch);
    return;
  }
  const long long n8 = n / 8;   // 16-byte units of 8 bf16
  const long long per = (n8 + world - 1) / world;
  const long long lo = min(n8, per * rank), hi = min(n8, per * (rank + 1));
  constexpr int UNROLL = 8;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = lo + (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < hi; i0 += stride * UNROLL) {
    uint4 out[UNROLL];
    if (MULTIMEM) {
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long i = i0 + u * stride;
        if (i < hi) {
          __nv_bfloat16* a = mc_base + offset_elems + i * 8;
          asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                       : "=r"(out[u].x), "=r"(out[u].y), "=r"(out[u].z), "=r"(out[u].w) : "l"(a) : "memory");
        }
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long i = i0 + u * stride;
        if (i < hi) {
          __nv_bfloat16* a = mc_base + offset_elems + i * 8;
          asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(a), "r"(out[u].x),
                       "r"(out[u].y), "r"(out[u].z), "r"(out[u].w) : "memory");
        }
      }
    } else {
      float acc[UNROLL][8];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[u][j] = 0.f;
      for (int q = 0; q < world; ++q) {
        uint4 v[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const long long i = i0 + u * stride;
          v[u] = make_uint4(0, 0, 0, 0);
          if (i < hi) v[u] = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(peers.buf[q]) + offset_elems + i * 8);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
            acc[u][2 * j] += f.x;
            acc[u][2 * j + 1] += f.y;
          }
        }
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long i = i0 + u * stride;
        if (i < hi) {
          const uint4 o = make_uint4(pack_bf16(acc[u][0], acc[u][1]), pack_bf16(acc[u][2], acc[u][3]),
                                     pack_bf16(acc[u][4], acc[u][5]), pack_bf16(acc[u][6], acc[u][7]));
          for (int q = 0; q < world; ++q)
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(peers.buf[q]) + offset_elems + i * 8) = o;
        }
      }
    }
  }
  if (rank == 0 && blockIdx.x == 0 && threadIdx.x < (n & 7)) {
    const long long i = n8 * 8 + threadIdx.x;
    float acc = 0.f;
    for (int q = 0; q < world; ++q) acc += __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(peers.buf[q])[offset_elems + i]);
    for (int q = 0; q < world; ++q) reinterpret_cast<__nv_bfloat16*>(peers.buf[q])[offset_elems + i] = __float2bfloat16(acc);
  }
  cross_rank_barrier(peers, rank, world, 1, epoch, status, wait_ns);
  end_call(ctrl, epoch);
}

// ---------------------------------------------------------------------------------------------------------------
// Push variant of the two-shot all-reduce (plain peer stores only; used when no multicast mapping is available or wanted).
//
// A peer LOAD over NVLink costs a round trip of microseconds, so a kernel that pulls its slice from the peers needs
// megabytes of loads in flight to fill the link; peer STORES are posted and stream at link speed from a few dozen CTAs.
// Here every remote access is a store:
//   1. push      rank r copies slice q of its contribution into rank q's staging area (slot of source r), for every q != r
//   2. barrier   block b of every rank tells block b of every peer that its part of the pushes has landed
//   3. reduce    rank r sums its own slice and the staged copies (local reads), applies `scale`, writes the result into
//                its own tensor and pushes it into slice r of every peer's tensor
//   4. barrier   block b waits until every peer's block b has pushed its results
// Every block handles the same strided part of every slice on every rank, so block-level flags are enough. The staging
// area ((world - 1) slots of one slice) lives behind the data region of the symmetric workspace.
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void add_unit(float (&acc)[8], const uint4& v, bool bf16) {
  if (bf16) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
      acc[2 * j] += f.x;
      acc[2 * j + 1] += f.y;
    }
  } else {
    acc[0] += __uint_as_float(v.x);
    acc[1] += __uint_as_float(v.y);
    acc[2] += __uint_as_float(v.z);
    acc[3] += __uint_as_float(v.w);
  }
}

template <bool BF16>
__global__ void __launch_bounds__(512)
allreduce_push_kernel(Peers peers, long long offset_bytes, long long staging_off_bytes, long long n16, float scale, int rank,
                      int world, unsigned long long wait_ns, KernelStatus* status) {
  unsigned int* ctrl = peers.flags[rank] + CTRL_WORDS_OFFSET;
  const unsigned int epoch = begin_call(ctrl);
  const long long per = (n16 + world - 1) / world;           // 16-byte units per slice
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long first = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const uint4* mine = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(peers.buf[rank]) + offset_bytes);
  constexpr int UNROLL = 8;
  // 1. push my contribution to the other slices' owners
  for (int k = 1; k < world; ++k) {
    const int q = (rank + k) % world;
    const long long lo = min(n16, per * q), hi = min(n16, per * (q + 1));
    const int slot = rank < q ? rank : rank - 1;
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<char*>(peers.buf[q]) + staging_off_bytes) + (long long)slot * per;
    for (long long i0 = lo + first; i0 < hi; i0 += stride * UNROLL) {
      uint4 v[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long i = i0 + u * stride;
        if (i < hi) v[u] = mine[i];
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long i = i0 + u * stride;
        if (i < hi) dst[i - lo] = v[u];
      }
    }
  }
  // 2. the pushes of block b have landed everywhere / everybody's have landed here
  if (!cross_rank_barrier(peers, rank, world, 0, epoch, status, wait_ns)) {
    end_call(ctrl, epoch);
    return;
  }
  // 3. reduce my slice from local memory, write it here and push it to the peers
  {
    const long long lo = min(n16, per * rank), hi = min(n16, per * (rank + 1));
    const uint4* staged = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(peers.buf[rank]) + staging_off_bytes);
    for (long long i0 = lo + first; i0 < hi; i0 += stride * UNROLL) {
      float acc[UNROLL][8];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[u][j] = 0.f;
        const long long i = i0 + u * stride;
        if (i < hi) add_unit(acc[u], mine[i], BF16);
      }
      for (int sl = 0; sl < world - 1; ++sl) {
        uint4 v[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const long long i = i0 + u * stride;
          v[u] = make_uint4(0, 0, 0, 0);
          if (i < hi) v[u] = staged[(long long)sl * per + (i - lo)];
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) add_unit(acc[u], v[u], BF16);
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long i = i0 + u * stride;
        if (i < hi) {
          uint4 o;
          if (BF16) {
            o = make_uint4(pack_bf16(acc[u][0], acc[u][1]), pack_bf16(acc[u][2], acc[u][3]), pack_bf16(acc[u][4], acc[u][5]),
                           pack_bf16(acc[u][6], acc[u][7]));
          } else {
            o = make_uint4(__float_as_uint(acc[u][0] * scale), __float_as_uint(acc[u][1] * scale),
                           __float_as_uint(acc[u][2] * scale), __float_as_uint(acc[u][3] * scale));
          }
          for (int k = 0; k < world; ++k) {
            const int q = (rank + k) % world;
            reinterpret_cast<uint4*>(reinterpret_cast<char*>(peers.buf[q]) + offset_bytes)[i] = o;
          }
        }
      }
    }
  }
  // 4. every peer's results are in my tensor
  cross_rank_barrier(peers, rank, world, 1, epoch, status, wait_ns);
  end_call(ctrl, epoch);
}

// Stand-alone cross-rank barrier (one block): "every rank of the group reached this point of its stream".
__global__ void barrier_kernel(Peers peers, int rank, int world, unsigned long long wait_ns, KernelStatus* status) {
  unsigned int* ctrl = peers.flags[rank] + CTRL_WORDS_OFFSET;
  const unsigned int epoch = begin_call(ctrl);
  cross_rank_barrier(peers, rank, world, 0, epoch, status, wait_ns);
  end_call(ctrl, epoch);
}

// Owner-side reduction of the dK/dV partials of ring attention. Every rank q >= me holds, in its symmetric partial
// buffer, fp32 partial gradients for the K/V chunk of rank `me` at  base_q + offset_elems  laid out as
// [2 (dk, dv)][tokens][width]. The sums are written as bf16 to dk / dv (token strides dk_row / dv_row).
__global__ void __launch_bounds__(256)
reduce_dkv_kernel(Peers peers, long long offset_elems, int me, int world, long long tokens, int width,
                  __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv, long long dk_row, long long dv_row) {
  const long long per = tokens * width;           // elements of one of dk / dv
  const long long n4 = per / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < 2 * n4; i += (long long)gridDim.x * blockDim.x) {
    const int which = i >= n4;
    const long long e = (i - which * n4) * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int q = me; q < world; ++q) {
      const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(peers.buf[q]) + offset_elems + which * per + e);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    const long long tok = e / width;
    const int col = (int)(e - tok * width);
    __nv_bfloat16* dst = (which ? dv : dk) + tok * (which ? dv_row : dk_row) + col;
    uint2 o;
    o.x = pack_bf16(acc.x, acc.y);
    o.y = pack_bf16(acc.z, acc.w);
    *reinterpret_cast<uint2*>(dst) = o;
  }
}

// Copies `n_src` equally sized blocks that live in peers' memory (plain 16-byte peer loads, many in flight per thread) into
// one contiguous local buffer: dst[i * units .. (i + 1) * units) = src[i][0 .. units), units of 16 bytes. Ring attention uses
// it to bring every remote K/V chunk across NVLink exactly once; the attention kernel then reads local memory only.
struct GatherSrc {
  const uint4* p[MAX_RANKS];
};
__global__ void __launch_bounds__(256)
gather_peer_kernel(uint4* __restrict__ dst, GatherSrc src, int n_src, long long units) {
  constexpr int UNROLL = 8;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long total = units * n_src;
  for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < total; i0 += stride * UNROLL) {
    uint4 v[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long i = i0 + u * stride;
      if (i < total) {
        const int which = (int)(i / units);
        v[u] = src.p[which][i - which * units];
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long i = i0 + u * stride;
      if (i < total) dst[i] = v[u];
    }
  }
}

// Vocabulary-parallel cross entropy: every rank left (row max, sum-exp, target logit) of its vocabulary shard for n rows in
// its own symmetric buffer at `offset_bytes` as three fp32 vectors [3][n]. After a barrier each rank combines all ranks'
// triples itself (plain peer loads of 12 bytes per row and rank): lse = gmax + log(sum_r sumexp_r * exp(max_r - gmax)),
// tgt = sum_r tgt_r. Replaces two NCCL all-reduces per chunk (max, then sum) of [n]-sized vectors.
__global__ void __launch_bounds__(256)
ce_stats_combine_peers_kernel(Peers peers, long long offset_bytes, int world, long long n, float* __restrict__ lse,
                              float* __restrict__ tgt) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float m[MAX_RANKS], s[MAX_RANKS], t = 0.f, gmax = -INFINITY;
  for (int q = 0; q < world; ++q) {
    const float* base = reinterpret_cast<const float*>(reinterpret_cast<const char*>(peers.buf[q]) + offset_bytes);
    m[q] = base[i];
    s[q] = base[n + i];
    t += base[2 * n + i];
    gmax = fmaxf(gmax, m[q]);
  }
  float sum = 0.f;
  for (int q = 0; q < world; ++q) sum += s[q] * __expf(m[q] - gmax);
  lse[i] = gmax + __logf(sum);
  tgt[i] = t;
}

// Vocabulary-parallel embedding without a reduction: the weight shards live in symmetric memory, and every rank reads the row
// of each of its tokens straight from the shard of the rank that owns it (16-byte peer loads). out[t, :] = W_owner[id - first].
__global__ void __launch_bounds__(256)
embedding_gather_peers_kernel(const long long* __restrict__ ids, Peers shards, int world, long long rows_per_rank, int H8,
                              uint4* __restrict__ out) {
  const long long tok = blockIdx.x;
  const long long id = ids[tok];
  const int owner = (int)(id / rows_per_rank);
  uint4* dst = out + tok * (long long)H8;
  if (id < 0 || owner >= world) {
    for (int c = threadIdx.x; c < H8; c += blockDim.x) dst[c] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(shards.buf[owner]) + (id - owner * rows_per_rank) * (long long)H8;
  for (int c = threadIdx.x; c < H8; c += blockDim.x) dst[c] = src[c];
}

}  // namespace comm
}  // namespace pt

extern "C" int pt_embedding_gather_peers(const long long* ids, void* const* shard_ptrs, int world, long long rows_per_rank,
                                         long long T, int H, void* out, cudaStream_t st) {
  using namespace pt::comm;
  if (world < 1 || world > MAX_RANKS || H % 8 || rows_per_rank <= 0) return -10;
  if (T <= 0) return 0;
  Peers shards;
  for (int q = 0; q < MAX_RANKS; ++q) {
    shards.buf[q] = q < world ? shard_ptrs[q] : nullptr;
    shards.flags[q] = nullptr;
  }
  embedding_gather_peers_kernel<<<(unsigned)T, 256, 0, st>>>(ids, shards, world, rows_per_rank, H / 8, reinterpret_cast<uint4*>(out));
  pt_count_launches(1);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int pt_ce_stats_combine_peers(void* const* buf_ptrs, long long offset_bytes, int world, long long n, float* lse,
                                         float* tgt, cudaStream_t st) {
  using namespace pt::comm;
  if (world < 1 || world > MAX_RANKS || offset_bytes % 4) return -10;
  if (n <= 0) return 0;
  Peers peers;
  for (int q = 0; q < MAX_RANKS; ++q) {
    peers.buf[q] = q < world ? buf_ptrs[q] : nullptr;
    peers.flags[q] = nullptr;
  }
  ce_stats_combine_peers_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(peers, offset_bytes, world, n, lse, tgt);
  pt_count_launches(1);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int pt_gather_peer(void* dst, const void* const* src_ptrs, int n_src, long long bytes_each, cudaStream_t st) {
  using namespace pt::comm;
  if (n_src < 0 || n_src > MAX_RANKS || bytes_each % 16 || (reinterpret_cast<uintptr_t>(dst) & 15)) return -10;
  if (n_src == 0 || bytes_each == 0) return 0;
  GatherSrc src;
  for (int i = 0; i < MAX_RANKS; ++i) {
    src.p[i] = i < n_src ? reinterpret_cast<const uint4*>(src_ptrs[i]) : nullptr;
    if (i < n_src && (reinterpret_cast<uintptr_t>(src_ptrs[i]) & 15)) return -10;
  }
  const long long units = bytes_each / 16;
  long long blocks = (units * n_src + 256 * 8 - 1) / (256 * 8);
  if (blocks > 1184) blocks = 1184;
  gather_peer_kernel<<<(unsigned)blocks, 256, 0, st>>>(reinterpret_cast<uint4*>(dst), src, n_src, units);
  pt_count_launches(1);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Limit of every cross-rank wait of the peer-memory kernels (this file and the fused GEMM + all-reduce), in nanoseconds of
// the GPU's global timer. Process-wide; read at launch time (a captured CUDA graph keeps the value it was captured with).
static unsigned long long g_wait_ns = pt::comm::kDefaultWaitNs;
extern "C" void pt_set_wait_limit_ns(unsigned long long ns) { g_wait_ns = ns ? ns : pt::comm::kDefaultWaitNs; }
extern "C" unsigned long long pt_get_wait_limit_ns() { return g_wait_ns; }

extern "C" int pt_symm_barrier(void* const* flag_ptrs, int rank, int world, cudaStream_t st) {
  using namespace pt;
  using namespace pt::comm;
  if (world < 1 || world > MAX_RANKS) return -10;
  Peers peers;
  for (int q = 0; q < MAX_RANKS; ++q) {
    peers.buf[q] = nullptr;
    peers.flags[q] = q < world ? reinterpret_cast<unsigned int*>(flag_ptrs[q]) : nullptr;
  }
  if (rank < 0 || rank >= world) return -10;
  barrier_kernel<<<1, 32, 0, st>>>(peers, rank, world, g_wait_ns, reinterpret_cast<KernelStatus*>(pt_status_word()));
  pt_count_launches(1);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int pt_reduce_dkv_symm(void* const* buf_ptrs, long long offset_elems, int me, int world, long long tokens,
                                  int width, void* dk, void* dv, long long dk_row, long long dv_row, cudaStream_t st) {
  using namespace pt;
  using namespace pt::comm;
  if (world < 1 || world > MAX_RANKS || width % 4 || dk_row % 4 || dv_row % 4 || offset_elems % 4) return -10;
  Peers peers;
  for (int q = 0; q < MAX_RANKS; ++q) {
    peers.buf[q] = q < world ? buf_ptrs[q] : nullptr;
    peers.flags[q] = nullptr;
  }
  const long long n4 = tokens * width / 4 * 2;
  int grid = (int)((n4 + 255) / 256);
  if (grid > 1184) grid = 1184;
  if (grid < 1) grid = 1;
  reduce_dkv_kernel<<<grid, 256, 0, st>>>(peers, offset_elems, me, world, tokens, width, (__nv_bfloat16*)dk,
                                          (__nv_bfloat16*)dv, dk_row, dv_row);
  pt_count_launches(1);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// In-place all-reduce (sum, times `scale` for fp32) of `n` elements starting `offset_elems` elements into the data
// region of a symmetric buffer. buf_ptrs/flag_ptrs: `world` peer-mapped base pointers of the data and flag regions
// (flag region: 2 * 8 * 128 uint32, zero-initialised once). mc_ptr: multicast mapping of the data region or null.
// All ranks must issue the same sequence of calls on a workspace (the call counter lives in the flag region, see the top of
// this file). Offsets must be 16-byte aligned.
// staging_off_bytes > 0 (and mc_ptr null): the push variant, with a staging area of at least
// (world - 1) * ceil(n * elem_size / 16 / world) * 16 bytes at that byte offset from every rank's data base; n must then be a
// multiple of 16 bytes' worth of elements (the caller falls back to staging_off_bytes = 0 otherwise).
extern "C" int pt_allreduce_symm(void* const* buf_ptrs, void* const* flag_ptrs, void* mc_ptr, long long offset_elems,
                                 long long n, int is_bf16, float scale, int rank, int world,
                                 int num_blocks, long long staging_off_bytes, cudaStream_t st) {
  using namespace pt;
  using namespace pt::comm;
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || num_blocks < 1 || num_blocks > MAX_BLOCKS) return -10;
  if (n <= 0) return 0;
  if ((offset_elems * (is_bf16 ? 2 : 4)) % 16) return -11;
  Peers peers;
  for (int q = 0; q < MAX_RANKS; ++q) {
    peers.buf[q] = q < world ? buf_ptrs[q] : nullptr;
    peers.flags[q] = q < world ? reinterpret_cast<unsigned int*>(flag_ptrs[q]) : nullptr;
  }
  KernelStatus* status = reinterpret_cast<KernelStatus*>(pt_status_word());
  const int esize = is_bf16 ? 2 : 4;
  if (mc_ptr == nullptr && staging_off_bytes > 0 && world > 1) {
    if ((n * esize) % 16 || staging_off_bytes % 16) return -11;
    const long long n16 = n * esize / 16;
    if (is_bf16)
      allreduce_push_kernel<true><<<num_blocks, 512, 0, st>>>(peers, offset_elems * esize, staging_off_bytes, n16, scale, rank, world,
                                                              g_wait_ns, status);
    else
      allreduce_push_kernel<false><<<num_blocks, 512, 0, st>>>(peers, offset_elems * esize, staging_off_bytes, n16, scale, rank, world,
                                                               g_wait_ns, status);
    pt_count_launches(1);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
  }
  if (is_bf16) {
    if (mc_ptr)
      allreduce_bf16_kernel<true><<<num_blocks, 512, 0, st>>>(peers, (__nv_bfloat16*)mc_ptr, offset_elems, n, rank, world, g_wait_ns, status);
    else
      allreduce_bf16_kernel<false><<<num_blocks, 512, 0, st>>>(peers, nullptr, offset_elems, n, rank, world, g_wait_ns, status);
  } else {
    if (mc_ptr)
      allreduce_f32_kernel<true><<<num_blocks, 512, 0, st>>>(peers, (float*)mc_ptr, offset_elems, n, scale, rank, world, g_wait_ns, status);
    else
      allreduce_f32_kernel<false><<<num_blocks, 512, 0, st>>>(peers, nullptr, offset_elems, n, scale, rank, world, g_wait_ns, status);
  }
  pt_count_launches(1);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

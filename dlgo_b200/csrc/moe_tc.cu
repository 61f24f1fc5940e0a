// Grouped contraction of routed experts on the tensor cores (tcgen05), in bfloat16: prompts, and decode steps of
// a couple of dozen (token, choice) pairs and more.
//
// Rows are (token, choice) pairs sorted by expert (the plan of moe.cu, tiles of 128 rows): tile t belongs to
// expert e = tile_expert[t] and covers sorted rows row0 .. row0 + 127, of which the first
// offsets[e + 1] - row0 are the expert's (the rest belong to the next expert, or lie beyond the last pair: they
// are computed and never stored).
//
//   out[o(r)][n] = act( sum_k A[r][k] * W[e][n][k] )
//
// A [rows, K] holds the rows in sorted order (moe_gather_rows copies the tokens' rows there for the experts'
// first contraction; the second reads the first one's output, which is written in sorted order).  W is the
// experts' weights stacked [experts * N, K].  Both operands arrive by TMA (128-byte swizzle, zero fill beyond
// the tensors, no multicast) in a shared-memory ring; one thread issues tcgen05.mma into a 128 x BN fp32
// accumulator in tensor memory; four warps read it back (a lane per row), apply the activation in fp32 and
// store a row's 32 columns at a time: in the activation type or fp32, at row r or at row o_scatter[r].
// Warp 0 loads, warp 1 issues MMAs, warps 2-5 are the epilogue.  CTAs are persistent (a few per SM, each walking
// the items it is dealt).  Every wait is bounded and sets an error word.
#include "common.cuh"
#include "tcgen05.cuh"

namespace dlgo {

using namespace sm100;

constexpr int GT_M = 128, GT_K = 64, GT_UMMA_K = 16, GT_THREADS = 192;
enum { GT_ACT_NONE = 0, GT_ACT_RELU2 = 1, GT_ACT_SILU = 2, GT_ACT_GELU_TANH = 3,
       // W's rows come in blocks of 16 gate rows followed by their 16 up rows: 32 columns of the accumulator give 16
       // columns silu(gate) * up of an output that is N / 2 wide (N a multiple of 32; single-CTA tiles only)
       GT_ACT_SWIGLU16 = 4 };

__device__ int g_moe_tc_error = 0;

struct GroupedTcParams {
  const int* offsets;
  const int* tile_expert;
  const int* tile_row0;
  const int* n_tiles;
  const int* o_scatter;     // null: sorted row r is row r of out
  void* out;
  long long ldo;
  int out_f32, act, N, K, stages;
  int nacc;                 // accumulators per CTA in tensor memory (1 or 2; the persistent single-CTA kernel)
};

__device__ __forceinline__ float gt_act(float v, int act) {
  switch (act) {
    case GT_ACT_RELU2: { const float r = fmaxf(v, 0.f); return r * r; }
    case GT_ACT_SILU: return v / (1.f + __expf(-v));
    case GT_ACT_GELU_TANH: return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    default: return v;
  }
}

// Persistent: a few CTAs per SM, each walking the work items (row tile, block of BN columns) it is dealt
// round-robin, columns first so that neighbouring CTAs read the same expert's weight tile at the same time.  The
// loader runs ahead into the next item's tiles while the epilogue warps empty the accumulator, and the MMAs of the
// next item start as soon as the accumulator has been read into registers.
template <int BN>
__global__ void __launch_bounds__(GT_THREADS)
moe_gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   const __grid_constant__ GroupedTcParams p) {
  constexpr int A_BYTES = GT_M * GT_K * 2, B_BYTES = BN * GT_K * 2, STAGE = A_BYTES + B_BYTES;
  extern __shared__ uint8_t gt_smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)gt_smem_raw + 1023) & ~(uintptr_t)1023);
  const int STAGES = p.stages;
  uint64_t* full = (uint64_t*)(smem + STAGES * STAGE);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;      // [2]
  uint64_t* acc_empty = acc_full + 2;       // [2]
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  const int NACC = p.nacc;                  // with two, the MMAs of the next item run under this item's epilogue
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  pdl_wait();                       // the plan and the rows are written by earlier kernels of the step
  const int n_tiles = *p.n_tiles;
  const int n_blocks = (p.N + BN - 1) / BN;
  const int n_items = n_tiles * n_blocks;
  if ((int)blockIdx.x >= n_items) return;   // before anything is allocated
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nkb = (p.K + GT_K - 1) / GT_K;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, NACC * BN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // Only now may the next kernel of the stream be scheduled: a tensor-core kernel allocates tensor memory in its
  // prologue and then waits for this grid; were it resident before this CTA holds its own columns, the two could
  // wait for each other.  (A grid's dependents start once every CTA of it has got here or has left.)
  pdl_launch_dependents();

  if (warp == 0) {
    if (elect_one()) {
      int it = 0;
      bool live = true;
      for (int item = blockIdx.x; item < n_items && live; item += gridDim.x) {
        const int tile = item % n_tiles, nb = item / n_tiles;
        const int e = p.tile_expert[tile], row0 = p.tile_row0[tile];
        for (int i = 0; i < nkb; ++i, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (it >= STAGES && !mbar_wait(&empty[s], ph ^ 1, abort_flag)) { live = false; break; }
          uint8_t* a_dst = smem + s * STAGE;
          mbar_expect_tx(&full[s], STAGE);
          tma_load_2d(a_dst, &map_a, &full[s], i * GT_K, row0);
          tma_load_2d(a_dst + A_BYTES, &map_b, &full[s], i * GT_K, e * p.N + nb * BN);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(GT_M, BN);
      int it = 0, j = 0;
      bool live = true;
      for (int item = blockIdx.x; item < n_items && live; item += gridDim.x, ++j) {
        // the epilogue warps have read this accumulator's previous item into registers
        const int b = NACC == 2 ? (j & 1) : 0, u = NACC == 2 ? (j >> 1) : j;
        if (u >= 1 && !mbar_wait(&acc_empty[b], (u - 1) & 1, abort_flag)) break;
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + (uint32_t)(b * BN);
        for (int i = 0; i < nkb; ++i, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full[s], ph, abort_flag)) { live = false; break; }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + s * STAGE);
          const uint64_t da = umma_desc_k_sw128(a_addr);
          const uint64_t db = umma_desc_k_sw128(a_addr + A_BYTES);
#pragma unroll
          for (int k = 0; k < GT_K / GT_UMMA_K; ++k) umma_bf16(tmem_d, da + 2 * k, db + 2 * k, idesc, (i | k) != 0);
          umma_commit(&empty[s]);
        }
        if (live) umma_commit(&acc_full[b]);
      }
    }
  } else {
    const int quarter = warp & 3;                 // warp w may touch tensor-memory lanes 32 * (w % 4) .. + 31
    const int r_in = quarter * 32 + lane;
    int j = 0;
    for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++j) {
      const int tile = item % n_tiles, nb = item / n_tiles;
      const int e = p.tile_expert[tile], row0 = p.tile_row0[tile];
      const int nr = min(GT_M, p.offsets[e + 1] - row0);
      const int n0 = nb * BN;
      const bool mine = r_in < nr;
      long long dst_row = 0;
      if (mine) dst_row = (p.o_scatter != nullptr ? p.o_scatter[row0 + r_in] : (row0 + r_in)) * p.ldo;
      const int b = NACC == 2 ? (j & 1) : 0, u = NACC == 2 ? (j >> 1) : j;
      if (!mbar_wait(&acc_full[b], u & 1, abort_flag)) break;
      tc_fence_after_sync();
      const uint32_t tmem_d = tmem_base + (uint32_t)(b * BN);
      // a lane per row, 32 columns at a time straight from tensor memory to global memory (a row's 32 columns
      // are 64 or 128 contiguous bytes); the accumulator is handed back as soon as its last columns are in registers
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        const bool last = c0 + 32 >= BN || n0 + c0 + 32 >= p.N;
        if (n0 + c0 >= p.N) break;                // (uniform over the warp)
        float v[32];
        tmem_ld_32x32(tmem_d + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
        tmem_ld_wait();
        if (last) {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[b]);
        }
        if (!mine) continue;
        if (p.act == GT_ACT_SWIGLU16) {              // (N is a multiple of 32: no ragged edge)
          const int col = (n0 + c0) >> 1;
#pragma unroll
          for (int q = 0; q < 16; ++q) v[q] = v[q] / (1.f + __expf(-v[q])) * v[q + 16];
          if (p.out_f32) {
            float* dst = (float*)p.out + dst_row + col;
#pragma unroll
            for (int q = 0; q < 16; ++q) dst[q] = v[q];
          } else {
            __nv_bfloat16* dst = (__nv_bfloat16*)p.out + dst_row + col;
            if (((uintptr_t)dst & 15) == 0) {
#pragma unroll
              for (int q = 0; q < 16; q += 8) {
                uint4 o;
                __nv_bfloat162 b0 = __floats2bfloat162_rn(v[q], v[q + 1]), b1 = __floats2bfloat162_rn(v[q + 2], v[q + 3]);
                __nv_bfloat162 b2 = __floats2bfloat162_rn(v[q + 4], v[q + 5]), b3 = __floats2bfloat162_rn(v[q + 6], v[q + 7]);
                o.x = *reinterpret_cast<unsigned*>(&b0); o.y = *reinterpret_cast<unsigned*>(&b1);
                o.z = *reinterpret_cast<unsigned*>(&b2); o.w = *reinterpret_cast<unsigned*>(&b3);
                *reinterpret_cast<uint4*>(dst + q) = o;
              }
            } else {
#pragma unroll
              for (int q = 0; q < 16; ++q) dst[q] = __float2bfloat16_rn(v[q]);
            }
          }
          continue;
        }
#pragma unroll
        for (int q = 0; q < 32; ++q) v[q] = gt_act(v[q], p.act);
        const int col = n0 + c0;
        if (p.out_f32) {
          float* dst = (float*)p.out + dst_row + col;
          if (col + 32 <= p.N && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
            for (int q = 0; q < 32; q += 4) *reinterpret_cast<float4*>(dst + q) = make_float4(v[q], v[q + 1], v[q + 2], v[q + 3]);
          } else {
#pragma unroll
            for (int q = 0; q < 32; ++q)
              if (col + q < p.N) dst[q] = v[q];
          }
        } else {
          __nv_bfloat16* dst = (__nv_bfloat16*)p.out + dst_row + col;
          if (col + 32 <= p.N && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
            for (int q = 0; q < 32; q += 8) {
              uint4 o;
              __nv_bfloat162 b0 = __floats2bfloat162_rn(v[q], v[q + 1]), b1 = __floats2bfloat162_rn(v[q + 2], v[q + 3]);
              __nv_bfloat162 b2 = __floats2bfloat162_rn(v[q + 4], v[q + 5]), b3 = __floats2bfloat162_rn(v[q + 6], v[q + 7]);
              o.x = *reinterpret_cast<unsigned*>(&b0); o.y = *reinterpret_cast<unsigned*>(&b1);
              o.z = *reinterpret_cast<unsigned*>(&b2); o.w = *reinterpret_cast<unsigned*>(&b3);
              *reinterpret_cast<uint4*>(dst + q) = o;
            }
          } else {
#pragma unroll
            for (int q = 0; q < 32; ++q)
              if (col + q < p.N) dst[q] = __float2bfloat16_rn(v[q]);
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(&g_moe_tc_error, 1);
    // give tile loads that may still be in flight time to land before shared memory is handed on
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, NACC * BN);
  }
}

// The same on CTA pairs (cta_group::2) for prompts: a pair takes TWO row tiles of one expert (the plan's tiles have 256
// rows; CTA r of the pair owns rows 128 r .. 128 r + 127 of it) against ONE weight tile of BN columns of which each
// CTA fetches half, so a k-block costs a CTA 16 KB of rows and BN / 2 x 128 bytes of weights for 128 x BN x 64 of
// MMA work: twice the FLOPs per operand byte of a single CTA on a 128 x 128 tile.  The leader's MMA warp issues for
// both; barriers as in the dense pair kernel: `full` counts both CTAs' bytes in the leader, `empty` and `acc_full`
// are signalled in both CTAs by one commit, `acc_empty` collects all 256 epilogue threads in the leader.  A half
// without rows of the expert (the expert's last rows fill only the first half) fetches no rows and stores nothing.
template <int BN>
__global__ void __launch_bounds__(GT_THREADS)
moe_gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                        const __grid_constant__ GroupedTcParams p) {
  constexpr int HALF_N = BN / 2;
  constexpr int A_BYTES = GT_M * GT_K * 2, B_BYTES = HALF_N * GT_K * 2, STAGE = A_BYTES + B_BYTES;
  extern __shared__ uint8_t gt_smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)gt_smem_raw + 1023) & ~(uintptr_t)1023);
  const int STAGES = p.stages;
  uint64_t* full = (uint64_t*)(smem + STAGES * STAGE);     // used in the leader only
  uint64_t* empty = full + STAGES;                          // local in each CTA
  uint64_t* acc_full = empty + STAGES;                      // local in each CTA
  uint64_t* acc_empty = acc_full + 1;                       // used in the leader only (256 arrivals)
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  pdl_wait();                       // the plan and the rows are written by earlier kernels of the step
  const int n_tiles = *p.n_tiles;
  const int n_blocks = (p.N + BN - 1) / BN;
  const int n_items = n_tiles * n_blocks;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  if (pair >= n_items) return;      // both CTAs of the pair, before anything is allocated
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int nkb = (p.K + GT_K - 1) / GT_K;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 256);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, BN);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();               // both CTAs' barriers exist before anything arrives on them remotely
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // (dependents only now: see the single-CTA kernel)
  pdl_launch_dependents();

  if (warp == 0) {
    if (elect_one()) {
      int it = 0;
      bool live = true;
      for (int item = pair; item < n_items && live; item += n_pairs) {
        const int tile = item % n_tiles, nb = item / n_tiles;
        const int e = p.tile_expert[tile], row0 = p.tile_row0[tile];
        const int rows_left = p.offsets[e + 1] - row0;                 // of the expert, from this tile on
        const bool peer_has = rows_left > GT_M, mine_has = rank == 0 || peer_has;
        for (int i = 0; i < nkb; ++i, ++it) {
          const int s = it % STAGES;
          if (it >= STAGES && !mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, abort_flag)) { live = false; break; }
          uint8_t* a_dst = smem + s * STAGE;
          // the leader's barrier counts the bytes of both CTAs' loads
          const uint32_t bar = map_to_cta(smem_u32(&full[s]), 0);
          if (rank == 0) mbar_expect_tx(&full[s], (peer_has ? 2 * A_BYTES : A_BYTES) + 2 * B_BYTES);
          if (mine_has) tma_load_2d_pair(a_dst, &map_a, bar, i * GT_K, row0 + (int)rank * GT_M);
          tma_load_2d_pair(a_dst + A_BYTES, &map_b, bar, i * GT_K, e * p.N + nb * BN + (int)rank * HALF_N);
        }
      }
    }
  } else if (warp == 1) {
    if (rank == 0 && elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(2 * GT_M, BN);
      int it = 0, j = 0;
      bool live = true;
      for (int item = pair; item < n_items && live; item += n_pairs, ++j) {
        if (j >= 1 && !mbar_wait(acc_empty, (j - 1) & 1, abort_flag)) break;
        tc_fence_after_sync();
        for (int i = 0; i < nkb; ++i, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(&full[s], (it / STAGES) & 1, abort_flag)) { live = false; break; }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + s * STAGE);
          const uint64_t da = umma_desc_k_sw128(a_addr);
          const uint64_t db = umma_desc_k_sw128(a_addr + A_BYTES);
#pragma unroll
          for (int k = 0; k < GT_K / GT_UMMA_K; ++k) umma_bf16_pair(tmem_base, da + 2 * k, db + 2 * k, idesc, (i | k) != 0);
          umma_commit_pair(&empty[s]);       // both CTAs may refill the stage
        }
        umma_commit_pair(acc_full);          // both CTAs' epilogues may read the accumulator (or leave, if not live)
      }
    }
  } else {
    const int quarter = warp & 3;
    const int r_in = quarter * 32 + lane;
    const uint32_t acc_empty_leader = map_to_cta(smem_u32(acc_empty), 0);
    int j = 0;
    for (int item = pair; item < n_items; item += n_pairs, ++j) {
      const int tile = item % n_tiles, nb = item / n_tiles;
      const int e = p.tile_expert[tile], row0 = p.tile_row0[tile] + (int)rank * GT_M;
      const int nr = min(GT_M, p.offsets[e + 1] - row0);             // may be <= 0 for the second half
      const int n0 = nb * BN;
      const bool mine = r_in < nr;
      long long dst_row = 0;
      if (mine) dst_row = (p.o_scatter != nullptr ? p.o_scatter[row0 + r_in] : (row0 + r_in)) * p.ldo;
      if (!mbar_wait(acc_full, j & 1, abort_flag)) break;
      tc_fence_after_sync();
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        const bool last = c0 + 32 >= BN || n0 + c0 + 32 >= p.N;
        if (n0 + c0 >= p.N) break;                // (uniform over the warp)
        float v[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
        tmem_ld_wait();
        if (last) {
          tc_fence_before_sync();
          mbar_arrive_cluster(acc_empty_leader);   // every epilogue thread of both CTAs
        }
        if (!mine) continue;
#pragma unroll
        for (int q = 0; q < 32; ++q) v[q] = gt_act(v[q], p.act);
        const int col = n0 + c0;
        if (p.out_f32) {
          float* dst = (float*)p.out + dst_row + col;
          if (col + 32 <= p.N && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
            for (int q = 0; q < 32; q += 4) *reinterpret_cast<float4*>(dst + q) = make_float4(v[q], v[q + 1], v[q + 2], v[q + 3]);
          } else {
#pragma unroll
            for (int q = 0; q < 32; ++q)
              if (col + q < p.N) dst[q] = v[q];
          }
        } else {
          __nv_bfloat16* dst = (__nv_bfloat16*)p.out + dst_row + col;
          if (col + 32 <= p.N && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
            for (int q = 0; q < 32; q += 8) {
              uint4 o;
              __nv_bfloat162 b0 = __floats2bfloat162_rn(v[q], v[q + 1]), b1 = __floats2bfloat162_rn(v[q + 2], v[q + 3]);
              __nv_bfloat162 b2 = __floats2bfloat162_rn(v[q + 4], v[q + 5]), b3 = __floats2bfloat162_rn(v[q + 6], v[q + 7]);
              o.x = *reinterpret_cast<unsigned*>(&b0); o.y = *reinterpret_cast<unsigned*>(&b1);
              o.z = *reinterpret_cast<unsigned*>(&b2); o.w = *reinterpret_cast<unsigned*>(&b3);
              *reinterpret_cast<uint4*>(dst + q) = o;
            }
          } else {
#pragma unroll
            for (int q = 0; q < 32; ++q)
              if (col + q < p.N) dst[q] = __float2bfloat16_rn(v[q]);
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();               // nobody leaves while the other CTA may still signal or be read
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(&g_moe_tc_error, 1);
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, BN);
  }
}

// Rows of the step's tokens in sorted pair order: dst[r] = src[pair(r) / div] for the r < offsets[experts] rows
// that belong to an expert (16 bytes per thread and step).
__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(const uint4* __restrict__ src, long long src_ld16, uint4* __restrict__ dst, int row16,
                       const int* __restrict__ sorted_pair, const int* __restrict__ total, int div, int max_rows,
                       const float* __restrict__ pair_scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int n = min(*total, max_rows);
  const long long items = (long long)n * row16;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < items; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / row16), c = (int)(i - (long long)r * row16);
    const int pair = sorted_pair[r];
    uint4 v = src[(long long)(pair / div) * src_ld16 + c];
    if (pair_scale != nullptr) {
      // bfloat16 rows whose pair brings a factor: the product in fp32, rounded once
      const float f = pair_scale[pair];
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 a = __bfloat1622float2(h[k]);
        h[k] = __floats2bfloat162_rn(a.x * f, a.y * f);
      }
    }
    dst[(long long)r * row16 + c] = v;
  }
}

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// [rows, K] bf16, row stride ld elements; box = 64 columns x box_rows rows, 128-byte swizzle, zero fill
int make_map(CUtensorMap* m, const void* base, long long rows, int K, long long ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return DLGO_ERR_DRIVER;
  if (((uintptr_t)base & 15) != 0 || (ld % 8) != 0) return DLGO_ERR_ALIGN;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)GT_K, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? DLGO_OK : DLGO_ERR_DRIVER;
}

template <int BN>
int launch_grouped(const CUtensorMap& ma, const CUtensorMap& mb, GroupedTcParams p, int max_tiles, int ring_default_kb,
                   cudaStream_t stream) {
  constexpr int STAGE = (GT_M + BN) * GT_K * 2;
  const int nkb = (p.K + GT_K - 1) / GT_K;
  // a small ring, so that several CTAs share an SM (one's epilogue and start-up under the others' MMAs): measured on a
  // B200 (width 2,048, 56 experts of 1,024, 8 chosen; prompt of 2,048 tokens / decode step at batch 8, ms): tiles 256
  // wide with 100 KB 3.29 / 0.734, with 150 KB 3.91 / 0.801; 128 wide with 100 KB 3.32 / 0.668, with 66 KB (two
  // stages, three CTAs an SM) 3.16 / 0.629; 64 wide with 75 KB (three stages, three CTAs an SM) 3.29 / 0.597.  So
  // prompts take 128 x 128 tiles and steps of few rows 128 x 64 (measured with one tile per CTA; with persistent
  // CTAs the order is the same: prompt tok/s / decode ms, 128 wide two stages 689 k / 0.578, 256 wide two stages 670 k
  // / 0.644, 64 wide three stages 658 k / 0.542).  DLGO_MOE_TC_RING_KB, DLGO_MOE_TC_BN (64, 128, 256) and
  // DLGO_MOE_TC_CTAS_PER_SM override.
  static const int ring_env = [] { const char* e = getenv("DLGO_MOE_TC_RING_KB"); return e ? atoi(e) : 0; }();
  const int ring_kb = ring_env > 0 ? ring_env : ring_default_kb;
  int stages = (ring_kb * 1024) / STAGE;
  if (stages > 8) stages = 8;
  if (stages > nkb) stages = nkb;
  if (stages < 2) stages = 2;
  p.stages = stages;
  const int smem = stages * STAGE + 1024 + 256;
  if (smem > 227 * 1024) return DLGO_ERR_SIZE;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(moe_gemm_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  // as many CTAs as are resident at once (what shared memory allows per SM), or fewer where the items are fewer
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  // two accumulators (the next item's MMAs under this item's epilogue) where tensor memory still allows three CTAs
  // per SM, i.e. on the 64-wide tiles of small steps: 0.545 -> 0.535 ms a decode step at batch 8; on 128-wide tiles
  // they cost a resident CTA and prompts lose (690 k -> 671 k tok/s).  DLGO_MOE_TC_NACC (1, 2) overrides.
  static const int nacc_env = [] { const char* e = getenv("DLGO_MOE_TC_NACC"); return e ? atoi(e) : 0; }();
  p.nacc = BN > 128 ? 1 : (nacc_env == 1 || nacc_env == 2 ? nacc_env : (BN == 64 ? 2 : 1));
  int per_sm = (227 * 1024) / (smem + 1024);
  const int by_tmem = 512 / (p.nacc * BN);
  if (per_sm > by_tmem) per_sm = by_tmem;
  if (per_sm < 1) per_sm = 1;
  static const int per_sm_env = [] { const char* e = getenv("DLGO_MOE_TC_CTAS_PER_SM"); return e ? atoi(e) : 0; }();
  if (per_sm_env > 0 && per_sm_env < per_sm) per_sm = per_sm_env;
  const long long items = (long long)max_tiles * ((p.N + BN - 1) / BN);
  const long long want = (long long)sms * per_sm;
  dim3 grid((unsigned)(items < want ? items : want));
  launch_kernel(moe_gemm_tc_kernel<BN>, grid, dim3(GT_THREADS), (size_t)smem, stream, ma, mb, p);
  return launch_status();
}

int launch_grouped_pair(const CUtensorMap& ma, const CUtensorMap& mb, GroupedTcParams p, int max_tiles,
                        cudaStream_t stream) {
  constexpr int BN = 256;
  constexpr int STAGE = (GT_M + BN / 2) * GT_K * 2;
  static const int ring_kb = [] { const char* e = getenv("DLGO_MOE_TC_PAIR_RING_KB"); return e ? atoi(e) : 96; }();
  int stages = (ring_kb * 1024) / STAGE;
  if (stages > 8) stages = 8;
  if (stages < 2) stages = 2;
  p.stages = stages;
  const int smem = stages * STAGE + 1024 + 256;
  if (smem > 227 * 1024) return DLGO_ERR_SIZE;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaError_t e = cudaFuncSetAttribute(moe_gemm_tc_pair_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) { sms = 0; return (int)e; }
  }
  int per_sm = (227 * 1024) / (smem + 1024);
  if (per_sm > 512 / BN) per_sm = 512 / BN;
  if (per_sm < 1) per_sm = 1;
  const long long items = (long long)max_tiles * ((p.N + BN - 1) / BN);
  long long pairs = (long long)sms * per_sm / 2;
  if (items < pairs) pairs = items;
  launch_kernel_cluster(moe_gemm_tc_pair_kernel<BN>, dim3((unsigned)(2 * pairs)), dim3(GT_THREADS), (size_t)smem, stream,
                        dim3(2, 1, 1), ma, mb, p);
  return launch_status();
}

}  // namespace
}  // namespace dlgo

using namespace dlgo;

// 1 if the tensor-core kernel takes these sizes (bfloat16 only): 16-byte rows for TMA.
DLGO_EXPORT int dlgo_moe_gemm_tc_takes(int N, int K) { return (N > 0 && K > 0 && K % 8 == 0) ? 1 : 0; }

// A [a_rows, K] bf16 (row stride lda) in sorted row order; W [experts * N, K] bf16 contiguous; the plan's tiles
// have 128 rows (one CTA per tile at a time) or 256 (CTA pairs).  out: bf16 or fp32 (out_f32), row stride ldo, rows r
// or o_scatter[r].
DLGO_EXPORT int dlgo_moe_gemm_tc(const void* A, long long a_rows, long long lda, const void* W, int experts, void* out,
                                 long long ldo, const int* o_scatter, const int* offsets, const int* tile_expert,
                                 const int* tile_row0, const int* n_tiles, int max_tiles, int tile_rows, int N, int K,
                                 int act, int out_f32, cudaStream_t stream) {
  if (max_tiles <= 0 || max_tiles > 65535 || a_rows <= 0 || experts <= 0) return DLGO_ERR_SIZE;
  if (!dlgo_moe_gemm_tc_takes(N, K)) return DLGO_ERR_SIZE;
  if (act == GT_ACT_SWIGLU16 && (N % 32 != 0 || tile_rows != GT_M)) return DLGO_ERR_SIZE;
  CUtensorMap ma, mb;
  if (tile_rows == 256) {
    // CTA pairs: each CTA fetches its 128 rows and half of a weight tile of 256 columns
    int st = make_map(&ma, A, a_rows, K, lda, GT_M);
    if (st != DLGO_OK) return st;
    st = make_map(&mb, W, (long long)experts * N, K, K, 128);
    if (st != DLGO_OK) return st;
    GroupedTcParams p{offsets, tile_expert, tile_row0, n_tiles, o_scatter, out, ldo, out_f32, act, N, K, 0, 1};
    return launch_grouped_pair(ma, mb, p, max_tiles, stream);
  }
  if (tile_rows != GT_M) return DLGO_ERR_SIZE;
  static const int force_bn = [] { const char* e = getenv("DLGO_MOE_TC_BN"); return e ? atoi(e) : 0; }();
  const int bn = force_bn == 64 || force_bn == 128 || force_bn == 256 ? force_bn : (a_rows <= 2048 ? 64 : 128);
  int st = make_map(&ma, A, a_rows, K, lda, GT_M);
  if (st != DLGO_OK) return st;
  st = make_map(&mb, W, (long long)experts * N, K, K, bn);
  if (st != DLGO_OK) return st;
  GroupedTcParams p{offsets, tile_expert, tile_row0, n_tiles, o_scatter, out, ldo, out_f32, act, N, K, 0, 1};
  if (bn == 256) return launch_grouped<256>(ma, mb, p, max_tiles, 100, stream);
  if (bn == 64) return launch_grouped<64>(ma, mb, p, max_tiles, 75, stream);
  return launch_grouped<128>(ma, mb, p, max_tiles, 66, stream);
}

// dst[r][:] = src[sorted_pair[r] / div][:] for the rows that belong to an expert; rows of `row_bytes` (a multiple of 16).
// `pair_scale` (fp32, one number per pair; rows of bfloat16 only): the row is multiplied by its pair's number.
DLGO_EXPORT int dlgo_moe_gather_rows(const void* src, long long src_ld_bytes, void* dst, int row_bytes,
                                     const int* sorted_pair, const int* total, int div, int max_rows,
                                     const float* pair_scale, cudaStream_t stream) {
  if (max_rows <= 0) return DLGO_OK;
  if (row_bytes <= 0 || row_bytes % 16 || src_ld_bytes % 16 || div <= 0 || ((uintptr_t)src & 15) || ((uintptr_t)dst & 15))
    return DLGO_ERR_ALIGN;
  const long long items = (long long)max_rows * (row_bytes / 16);
  long long want = (items + 255) / 256;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  launch_kernel(moe_gather_rows_kernel, dim3(blocks), dim3(256), 0, stream, (const uint4*)src, src_ld_bytes / 16,
                (uint4*)dst, row_bytes / 16, sorted_pair, total, div, max_rows, pair_scale);
  return launch_status();
}

// The error word (1: a bounded wait ran out), cleared by the read.
DLGO_EXPORT int dlgo_moe_tc_error() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, dlgo::g_moe_tc_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(dlgo::g_moe_tc_error, &zero, sizeof(int));
  return v;
}

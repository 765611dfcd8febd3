// CTA-pair variant of the persistent bf16 GEMM: two CTAs of a cluster compute one 256 x 256 output tile with
// tcgen05.mma.cta_group::2.  Each CTA stages its own 128 rows of A and only HALF of the B tile (128 rows), and holds
// its own 128 x 256 accumulator in TMEM; the tensor core of each SM reads the other half of B from the peer's shared
// memory.  Per output element this moves a third less shared-memory operand traffic than the one-CTA kernel, whose
// limiter that traffic is.
//
// Protocol (rank 0 of the pair is the leader):
//   * both CTAs run a TMA producer; loads carry .cta_group::2 (no multicast) and signal the LEADER's `full` barrier,
//     on which the leader's producer has posted the byte count of both CTAs;
//   * only the leader issues MMAs; it commits to the `empty` / `tfull` barriers of both CTAs with one commit per CTA
//     (the peer's barrier is addressed through its shared::cluster address);
//   * both CTAs run the TMA-store epilogue on their own accumulator rows and arrive on the leader's `tempty` barrier.
// Every wait is bounded; both CTAs always reach the closing cluster barrier.
#include "gemm_epilogue.cuh"
#include "himuon.h"
#include "sm100_common.cuh"
#include "tma_host.h"


namespace himuon {

constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;   // clears the CTA-rank bit of a shared::cluster address (pair leader)

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma2_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at shared::cluster address `bar_addr` once all MMAs issued so far by this thread are done.
__device__ __forceinline__ void umma2_commit(uint32_t bar_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_addr) : "memory");
}
// TMA load issued by either CTA of the pair; completion bytes go to the LEADER's barrier.
__device__ __forceinline__ void tma2_load_3d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(smem_u32(bar) & kPeerBitMask), "r"(x), "r"(y), "r"(z)
      : "memory");
}

constexpr int BN2 = 256;     // tile width
constexpr int BNH = 128;     // rows of B staged by each CTA

template <int STAGES, bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(256, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmW, GemmDev p) {
  constexpr uint32_t A_BYTES = BM * BK * 2;
  constexpr uint32_t B_BYTES = BNH * BK * 2;
  constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t CHUNK_BYTES = BK * 128;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align_up_1024(smem_raw);
  uint8_t* sC = smem + STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sC + 2 * SLAB_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tfull = bars + 2 * STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 8);      // four epilogue warps in each CTA of the pair
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 2) tmem_alloc2(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_per_batch = p.tiles_m * p.tiles_n;
  const int pair = blockIdx.x >> 1;
  const int n_pairs = gridDim.x >> 1;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      WorkCursor cur(p, pair, n_pairs);
      WorkItem w;
      while (ok && cur.next(w)) {
        const int tile = w.tile;
        const int b = tile / tiles_per_batch;
        const int r = tile - b * tiles_per_batch;
        const int mt = r % p.tiles_m;
        const int nt = r / p.tiles_m;
        const int m0 = mt * 2 * BM + static_cast<int>(rank) * BM;
        const int n0 = nt * BN2 + static_cast<int>(rank) * BNH;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status, 1)) { ok = false; break; }
          uint8_t* sA = smem + stage * STAGE_BYTES;
          uint8_t* sB = sA + A_BYTES;
          if (leader) mbar_expect_tx(&full[stage], 2 * STAGE_BYTES);
          if (!A_MN) {
            tma2_load_3d(sA, &tmA, &full[stage], kb * BK, m0, b);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma2_load_3d(sA + j * CHUNK_BYTES, &tmA, &full[stage], m0 + j * 64, kb * BK, b);
          }
          if (!B_MN) {
            tma2_load_3d(sB, &tmB, &full[stage], kb * BK, n0, b);
          } else {
#pragma unroll
            for (int j = 0; j < BNH / 64; ++j) tma2_load_3d(sB + j * CHUNK_BYTES, &tmB, &full[stage], n0 + j * 64, kb * BK, b);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = umma_idesc_bf16(2 * BM, BN2, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      WorkCursor cur(p, pair, n_pairs);
      WorkItem w;
      while (ok && cur.next(w)) {
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag, p.status, 2)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN2);
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, p.status, 2)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_base = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t b_base = a_base + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = A_MN ? umma_smem_desc(a_base + k * 2048, CHUNK_BYTES, 1024)
                                        : umma_smem_desc(a_base + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? umma_smem_desc(b_base + k * 2048, CHUNK_BYTES, 1024)
                                        : umma_smem_desc(b_base + k * 32, 16, 1024);
            umma2_ss(d_tmem, adesc, bdesc, idesc, (kb > w.kb0 || k > 0) ? 1u : 0u);
          }
          const uint32_t e_addr = smem_u32(&empty[stage]);
          umma2_commit(e_addr);                    // this CTA's producer
          umma2_commit(map_to_cta(e_addr, 1));     // the peer's producer
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        const uint32_t f_addr = smem_u32(&tfull[acc]);
        umma2_commit(f_addr);
        umma2_commit(map_to_cta(f_addr, 1));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ epilogue (both CTAs, own 128 accumulator rows)
    const int ew = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t slab_seq = 0;
    const bool issuer = (threadIdx.x == 128);
    if (issuer) tma_prefetch_desc(&tmC);
    WorkCursor cur(p, pair, n_pairs);
    WorkItem w;
    while (cur.next(w)) {
      const int tile = w.tile;
      const int b = tile / tiles_per_batch;
      const int r = tile - b * tiles_per_batch;
      const int mt = r % p.tiles_m;
      const int nt = r / p.tiles_m;
      if (!mbar_wait(&tfull[acc], acc_phase, abort_flag, p.status, 3)) break;
      tc_fence_after();
      const int row_in_tile = ew * 32 + lane;
      const int m0 = mt * 2 * BM + static_cast<int>(rank) * BM;
      const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + static_cast<uint32_t>(acc * BN2);
      const long long aux_row = static_cast<long long>(b) * p.strideAux + static_cast<long long>(m0 + row_in_tile) * p.ldaux;
      if (w.split) {
        // K-slice of a last-wave tile: add the fp32 partial into the scratch tile (rows tail*256 + rank*128 ..);
        // a follow-up kernel applies the epilogue to the complete sums
        epilogue_tile_tma<BN2, true>(&tmW, sC, t_acc, row_in_tile, w.tail * 2 * BM + static_cast<int>(rank) * BM, 0, 0, nullptr, 0,
                                     1 << 30, BN2, 1.f, 0.f, 0, slab_seq, issuer, true);
      } else if (m0 < p.M) {              // uniform: the second CTA of a ragged last row block has nothing to store
        if (p.reduce_out && p.out_fp32)   // C += alpha*acc without reading C: the L2 adds the staged slabs
          epilogue_tile_tma<BN2, true>(&tmC, sC, t_acc, row_in_tile, m0, nt * BN2, b, nullptr, 0, p.M, p.N, p.alpha,
                                       0.f, 0, slab_seq, issuer, true);
        else if (p.reduce_out)            // same for a bf16 C: the partial is rounded to bf16, then added in bf16
          epilogue_tile_tma<BN2, false>(&tmC, sC, t_acc, row_in_tile, m0, nt * BN2, b, nullptr, 0, p.M, p.N, p.alpha,
                                        0.f, 0, slab_seq, issuer, true);
        else if (p.out_fp32)
          epilogue_tile_tma<BN2, true>(&tmC, sC, t_acc, row_in_tile, m0, nt * BN2, b, p.aux, aux_row, p.M, p.N, p.alpha,
                                       p.beta, p.round_acc, slab_seq, issuer);
        else
          epilogue_tile_tma<BN2, false>(&tmC, sC, t_acc, row_in_tile, m0, nt * BN2, b, p.aux, aux_row, p.M, p.N, p.alpha,
                                        p.beta, p.round_acc, slab_seq, issuer);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty[acc]), 0));   // the leader owns the accumulator hand-off
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    if (issuer) tma_store_wait_all();      // reductions into the scratch tiles are complete before the kernel ends
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                  // neither CTA leaves while the other may still signal or read it
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, 512);
  }
}

// Second half of the split-K tail: turns the complete fp32 sums of the last-wave tiles into outputs (alpha, beta*aux,
// optional bf16 rounding point, cast) and leaves the scratch zeroed for the next launch.
template <typename T>
__global__ void __launch_bounds__(256)
gemm2_finish_kernel(float* __restrict__ ws, GemmDev p, int first_tail_tile, int n_tail) {
  const int tiles_per_batch = p.tiles_m * p.tiles_n;
  const long long per_tile = 256LL * 256 / 4;            // float4 groups per tile
  const long long total = per_tile * n_tail;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / per_tile);
    const int e = static_cast<int>(i - t * per_tile);
    const int r = e >> 6, c = (e & 63) * 4;
    float4* src = reinterpret_cast<float4*>(ws + (static_cast<long long>(t) * 256 + r) * 256 + c);
    const float4 v = *src;
    *src = make_float4(0.f, 0.f, 0.f, 0.f);
    const int tile = first_tail_tile + t;
    const int b = tile / tiles_per_batch;
    const int rr = tile - b * tiles_per_batch;
    const int row = (rr % p.tiles_m) * 256 + r;
    const int col = (rr / p.tiles_m) * 256 + c;
    if (row >= p.M) continue;
    const float vals[4] = {v.x, v.y, v.z, v.w};
    T* cp = reinterpret_cast<T*>(p.C) + static_cast<long long>(b) * p.strideC + static_cast<long long>(row) * p.ldc + col;
    const T* xp = p.aux ? reinterpret_cast<const T*>(p.aux) + static_cast<long long>(b) * p.strideAux +
                              static_cast<long long>(row) * p.ldaux + col
                        : nullptr;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (col + j >= p.N) break;
      float o = p.alpha * vals[j];
      if (xp) {
        if (p.round_acc) o = round_bf16(o);
        if (sizeof(T) == 2) o += p.beta * __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(xp)[j]);
        else o += p.beta * reinterpret_cast<const float*>(xp)[j];
      }
      if (sizeof(T) == 2) reinterpret_cast<__nv_bfloat16*>(cp)[j] = __float2bfloat16_rn(o);
      else reinterpret_cast<float*>(cp)[j] = o;
    }
  }
}

// fp32 scratch for the split-K tail of the pair kernel: up to kPairTailMax tiles of 256 x 256, zero between launches.
// One buffer per device, shared by every GEMM of that device (GEMMs that split must not overlap on different streams).
constexpr int kPairTailMax = 40;
static float* pair_scratch() {
  static float* per_device[64] = {nullptr};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (per_device[dev] == nullptr) {
    void* ptr = nullptr;
    const size_t bytes = static_cast<size_t>(kPairTailMax) * 256 * 256 * sizeof(float);
    if (cudaMalloc(&ptr, bytes) == cudaSuccess && cudaMemset(ptr, 0, bytes) == cudaSuccess) per_device[dev] = static_cast<float*>(ptr);
    else cudaGetLastError();
  }
  return per_device[dev];
}

template <int STAGES, bool A_MN, bool B_MN>
static void launch_gemm2(const GemmArgs& a, cudaStream_t stream) {
  constexpr uint32_t STAGE_BYTES = (BM + BNH) * BK * 2;
  constexpr size_t SMEM = 1024 + STAGES * STAGE_BYTES + 2 * SLAB_BYTES + 256;
  static_assert(SMEM <= 232448, "shared memory budget of one CTA exceeded");
  auto kern = gemm2_bf16_kernel<STAGES, A_MN, B_MN>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SMEM));
    attr_done = true;
  }
  uint64_t dimsA[3], strA[2], dimsB[3], strB[2];
  uint32_t boxA[3], boxB[3];
  if (!A_MN) { dimsA[0] = a.K; dimsA[1] = a.M; boxA[0] = BK; boxA[1] = BM; }
  else       { dimsA[0] = a.M; dimsA[1] = a.K; boxA[0] = 64; boxA[1] = BK; }
  dimsA[2] = a.batch; boxA[2] = 1;
  strA[0] = static_cast<uint64_t>(a.lda) * 2;
  strA[1] = a.batch > 1 ? static_cast<uint64_t>(a.strideA) * 2 : strA[0] * dimsA[1];
  if (!B_MN) { dimsB[0] = a.K; dimsB[1] = a.N; boxB[0] = BK; boxB[1] = BNH; }
  else       { dimsB[0] = a.N; dimsB[1] = a.K; boxB[0] = 64; boxB[1] = BK; }
  dimsB[2] = a.batch; boxB[2] = 1;
  strB[0] = static_cast<uint64_t>(a.ldb) * 2;
  strB[1] = a.batch > 1 ? static_cast<uint64_t>(a.strideB) * 2 : strB[0] * dimsB[1];
  const CUtensorMap tmA = make_tmap(a.A, 3, dimsA, strA, boxA, 2, true);
  const CUtensorMap tmB = make_tmap(a.B, 3, dimsB, strB, boxB, 2, true);
  const int esz = a.out_fp32 ? 4 : 2;
  const uint64_t dimsC[3] = {static_cast<uint64_t>(a.N), static_cast<uint64_t>(a.M), static_cast<uint64_t>(a.batch)};
  const uint64_t strC[2] = {static_cast<uint64_t>(a.ldc) * esz,
                            a.batch > 1 ? static_cast<uint64_t>(a.strideC) * esz : static_cast<uint64_t>(a.ldc) * esz * a.M};
  const uint32_t boxC[3] = {static_cast<uint32_t>(128 / esz), BM, 1};
  const CUtensorMap tmC = make_tmap(a.C, 3, dimsC, strC, boxC, esz, true);

  GemmDev p{};
  p.C = a.C; p.aux = a.aux;
  p.M = a.M; p.N = a.N; p.K = a.K; p.batch = a.batch;
  p.ldc = a.ldc; p.ldaux = a.ldaux; p.strideC = a.strideC; p.strideAux = a.strideAux;
  p.alpha = a.alpha; p.beta = a.beta; p.out_fp32 = a.out_fp32; p.round_acc = a.round_acc;
  p.tiles_m = (a.M + 2 * BM - 1) / (2 * BM);
  p.tiles_n = (a.N + BN2 - 1) / BN2;
  p.kblocks = (a.K + BK - 1) / BK;
  p.tma_store = 1;
  p.nslices = 1;
  p.reduce_out = (a.aux == a.C && a.beta == 1.f && !a.round_acc &&
                  a.ldaux == a.ldc && a.strideAux == a.strideC) ? 1 : 0;
  p.status = status_word_ptr();
  const long long total = static_cast<long long>(p.tiles_m) * p.tiles_n * a.batch;
  p.full_items = p.total_items = static_cast<int>(total);
  // Clusters that can be resident at once (GPCs with an odd number of free SMs leave one SM unpaired).
  static int max_pairs = 0;
  if (max_pairs == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(num_sms());
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = SMEM;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) == cudaSuccess && n > 0) max_pairs = n;
    else { cudaGetLastError(); max_pairs = num_sms() / 2; }
  }
  int cap = max_pairs;
  if (a.max_ctas > 0 && a.max_ctas / 2 < cap) cap = a.max_ctas / 2 > 0 ? a.max_ctas / 2 : 1;
  // Split the tiles of a mostly idle last wave along K: each K-slice adds its fp32 partial tile into a scratch tile
  // with TMA reductions and a small follow-up kernel applies the epilogue.
  CUtensorMap tmW = tmC;
  const int rem = static_cast<int>(total % cap);
  float* scratch = nullptr;
  // Accumulating fp32 outputs need no scratch to split a tile along K (every part just adds into C), so their work is
  // dealt out in equal contiguous (tile, k-block) ranges whenever whole tiles would not fill the last wave.
  const bool want_stream = p.reduce_out && total % cap != 0 && p.kblocks >= 8 &&
                           total * p.kblocks >= 8LL * cap;
  if (!want_stream && total > cap / 2 && rem > 0 && rem * 2 <= cap && rem <= kPairTailMax && p.kblocks >= 16 &&
      (scratch = pair_scratch()) != nullptr) {
    int sl = cap / rem;
    if (sl > p.kblocks / 8) sl = p.kblocks / 8;
    // worth it only when the K-blocks saved outweigh the fp32 reduction traffic and the second launch (~12 us)
    if (sl >= 2 && (sl - 1) * p.kblocks / sl >= 40) {
      p.nslices = sl;
      p.full_items = static_cast<int>(total) - rem;
      p.total_items = p.full_items + rem * sl;
      const uint64_t dimsW[3] = {256, static_cast<uint64_t>(kPairTailMax) * 256, 1};
      const uint64_t strW[2] = {256 * sizeof(float), static_cast<uint64_t>(kPairTailMax) * 256 * 256 * sizeof(float)};
      const uint32_t boxW[3] = {32, BM, 1};
      tmW = make_tmap(scratch, 3, dimsW, strW, boxW, 4, true);
    }
  }
  long long pairs = p.total_items < cap ? p.total_items : cap;
  if (want_stream) {
    p.stream_k = 1;
    pairs = cap;
  }
  kern<<<static_cast<int>(2 * pairs), 256, SMEM, stream>>>(tmA, tmB, tmC, tmW, p);
  if (p.nslices > 1) {
    const long long groups = 256LL * 256 / 4 * rem;
    const int blocks = static_cast<int>((groups + 255) / 256 < num_sms() * 4 ? (groups + 255) / 256 : num_sms() * 4);
    if (a.out_fp32) gemm2_finish_kernel<float><<<blocks, 256, 0, stream>>>(scratch, p, p.full_items, rem);
    else gemm2_finish_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(scratch, p, p.full_items, rem);
  }
}

// True when the pair kernel can run this problem and is expected to win: TMA-storable output, more than one CTA
// tile of rows, and a reduction long enough (K >= 2048) to amortise the 256-column epilogue; short-K batched
// products (the Newton-Schulz GEMMs) are faster on the one-CTA kernel.
bool gemm2_supported(const GemmArgs& a) {
  const int esz = a.out_fp32 ? 4 : 2;
  const int row_align = 16 / esz;
  return a.M > BM && a.N > 192 && a.K >= 2048 && (a.ldc % row_align == 0) && (a.batch == 1 || a.strideC % row_align == 0) &&
         (reinterpret_cast<uintptr_t>(a.C) % 16 == 0);
}

void gemm2_bf16(const GemmArgs& a, cudaStream_t stream) {
  const int sel = (a.a_mn ? 2 : 0) | (a.b_mn ? 1 : 0);
  switch (sel) {
    case 0: launch_gemm2<6, false, false>(a, stream); break;
    case 1: launch_gemm2<6, false, true>(a, stream); break;
    case 2: launch_gemm2<6, true, false>(a, stream); break;
    default: launch_gemm2<6, true, true>(a, stream); break;
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("himuon gemm (pair) launch failed: ") + cudaGetErrorString(e));
}

}  // namespace himuon

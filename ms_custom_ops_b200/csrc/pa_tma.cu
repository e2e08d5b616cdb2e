// Paged-attention decode for B200: persistent TMA-fed split-KV kernel.
//
// HBM-bound: every K/V byte of the context is read exactly once.  One
// persistent CTA per SM takes work items (sequence, kv head, q-row block, KV
// split) from a longest-first list by a ticket.  A producer warp streams K and V
// tiles of the paged cache into a ring of shared-memory stages with tiled TMA
// loads (cp.async.bulk.tensor, 128-byte swizzle, no multicast) that complete
// on mbarriers; the stream runs ahead across item boundaries, so the memory
// pipe never drains between items.  Each consumer warp owns 16 (or 32) tokens
// of a tile and keeps an independent online-softmax state (m, l, O) for the GQA
// group of q rows.
//
// The micro-tiles put the TOKENS on the M side of mma.sync m16n8k16 and the q
// rows on the N side (N = 8 per tile, one or two tiles), so a group of up to 8
// q rows costs no padding work:
//   S^T = K Q^T     A = K tile (ldmatrix),        B = Q^T (registers, loaded once per item)
//   O^T += V^T P^T  A = V^T   (ldmatrix.trans),   B = P^T (movmatrix of the probabilities)
// fp32 accumulation throughout.  int8 KV: bytes become fp16 in registers
// (xor 0x80, byte-permute into 0x6400|u = 1024 + u); for K the constant 1152
// is not removed because it shifts every score of a q row by the same amount,
// which the softmax cancels; for V it stays in the accumulators and
// 1152 * l is subtracted once per item.  The row sums l are accumulated by the
// tensor cores from the same rounded probabilities (a tile of ones in place
// of V^T).  k_descale is folded into Q once per item by a helper warp, v_descale /
// v_offset are applied once to the output.  At the end of an item the warps' states are
// merged through shared memory and written either as the final output (one split) or
// as an fp32 partial (m, l, O); the CTA that stores the last partial of a
// (sequence, kv head, q-row block) group merges the group's partials itself.
//
// Head dimensions: 128 (16-bit and int8 KV), 64 and 256 (16-bit KV).
// Algorithmic bytes per context token: 2 * head_dim * sizeof(kv) per kv head.
#include <cuda.h>

#include <type_traits>

#include "msco_common.cuh"
#include "pa_merge.cuh"
#include "pa_params.h"

namespace msco {
namespace {

constexpr float kNeg = -1.0e30f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr uint32_t kWaitLimit = 1u << 24;
constexpr int kDescInts = 12;  // work-item descriptor handed from the producer to the consumers

// D = head_dim, NT = number of 8-row tiles of the q group (1: up to 8 rows, 2: up to 16),
// SUBS = 16-token sub-tiles per consumer warp and tile.
template <int D, bool KV8, int NT, int SUBS> struct Cfg {
  static_assert(D == 64 || D == 128 || D == 256, "head_dim 64, 128 or 256");
  static_assert(!KV8 || D == 128, "int8 KV: head_dim 128");
  // rows of 128 bytes (int8 KV at head_dim 128, 16-bit KV at head_dim 64) with up to 8 q rows: two 16-token
  // sub-tiles per consumer warp (256-token tiles of 32 KB, two independent MMA chains per warp)
  static_assert((SUBS == 2) == ((KV8 || D == 64) && NT == 1), "sub-tiles per warp do not match the variant");
  static_assert(D != 256 || NT == 1, "head_dim 256: up to 8 q rows per item");
  static constexpr int kWarps = D == 256 ? 4 : 8;           // consumer warps
  static constexpr int kTile = kWarps * 16 * SUBS;          // tokens per tile
  static constexpr int kAux = KV8 ? 1 : 0;                  // helper warp that prepares Q (int8 KV)
  // warps: consumers, the producer, the warp that counts stored partials, (int8 KV) the Q-preparation warp
  static constexpr int kThreads = (kWarps + 2 + kAux) * 32;
  static constexpr int kConsumerThreads = kWarps * 32;
  static constexpr int kRowBytes = KV8 ? D : 2 * D;         // one token row of one head
  static constexpr int kBoxes = kRowBytes / 128;            // 128-byte TMA boxes per token row
  static constexpr int kStageBytes = kTile * kRowBytes;     // 16 / 32 KB
  static constexpr int kStages = D == 64 ? (NT == 1 ? 4 : 8) : (D == 256 ? 5 : (KV8 ? (NT == 1 ? 4 : 8) : (NT == 1 ? 5 : 4)));
  static constexpr int kRows = 8 * NT;
  static constexpr int kKSteps = D / 16;                    // 16-wide slices of the head dimension
  static constexpr int kMergeStride = D + 4;                // floats per merged row (bank-conflict padding)
  static constexpr int kMergeBufs = SUBS == 2 ? 2 : 1;      // two: no barrier between the items' merges
  static constexpr int kMergeBytes = kWarps * kRows * kMergeStride * 4;
  static constexpr int kMlBytes = kWarps * 16 * 2 * 4;      // [warp][16] float2
  static constexpr int kQSlotBytes = 16 * D * 2;
  static constexpr int kOffQ = kStages * kStageBytes;
  static constexpr int kOffQFrag = kOffQ + 2 * kQSlotBytes;         // int8 KV: scaled fp16 Q in fragment order
  static constexpr int kQFragBytes = KV8 ? NT * 4 * 32 * 16 + 128 : 0;  // [row tile][k-step pair][lane] uint4, then
                                                                         // 2 partial score offsets per q row (lse)
  static constexpr int kOffMerge = kOffQFrag + 2 * kQFragBytes;
  static constexpr int kOffMl = kOffMerge + kMergeBufs * kMergeBytes;
  static constexpr int kOffDesc = kOffMl + kMergeBufs * kMlBytes;   // 2 x kDescInts ints, 4 spare ints,
                                                                    // 4 x 8 ints: groups awaiting their merge
  static constexpr int kOffShift = kOffDesc + 2 * kDescInts * 4 + 16 + 4 * 8 * 4;  // 2 x 32 floats (lse, int8 KV)
  static constexpr int kOffBar = kOffShift + 2 * 32 * 4;            // mbarriers
  static constexpr int kNumBars = 2 * kStages + 8;
  static constexpr int kOffItemBase = kOffBar + kNumBars * 8 + 16;  // copy of the plan's item_base[]
  static constexpr int kItemBaseCap = 1024;                          // sequences (+1) that fit
  static constexpr int kSmemBytes = kOffItemBase + kItemBaseCap * 4;
  static constexpr int kDynSmem = kSmemBytes + 1024;                // slack for 1024-byte alignment
};

// int8x4 (already xor-ed with 0x80808080) -> fp16x2 {1024 + u_a, 1024 + u_b}; sel picks bytes a, b.
__device__ __forceinline__ uint32_t bytes_to_half2_biased(uint32_t x, uint32_t sel) {
  uint32_t h;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(h) : "r"(x), "r"(0x64646464u), "r"(sel));
  return h;
}
// transpose of an 8x8 matrix of 16-bit values held as one register per lane
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}

// additive mask element (decode shapes): NORM [batch, 1, ctx] (head stride 0), ALIBI [batch, heads, 1, ctx]
__device__ __forceinline__ float load_mask_elem(const void *mask, int dtype, int64_t idx) {
  if (dtype == MSCO_DTYPE_F16) return __half2float(__ldg(static_cast<const __half *>(mask) + idx));
  if (dtype == MSCO_DTYPE_BF16) return __bfloat162float(__ldg(static_cast<const __nv_bfloat16 *>(mask) + idx));
  return __ldg(static_cast<const float *>(mask) + idx);
}

template <typename T, int D, bool KV8, int NT, bool MASK, int SUBS, int PW>
__global__ void __launch_bounds__(Cfg<D, KV8, NT, SUBS>::kThreads, 1)
pa_tma_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, PaParams p,
              const __grid_constant__ PlanParamT<PW> pp) {
  using C = Cfg<D, KV8, NT, SUBS>;
  // fp16 arithmetic for int8 KV (integers up to 1279 are exact in fp16, not in bf16)
  using MT = typename std::conditional<KV8, __half, T>::type;
  constexpr int kTile = C::kTile;
  constexpr int kKS = C::kKSteps;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + C::kOffBar);
  uint64_t *full = bars, *empty = bars + C::kStages;
  uint64_t *qfull = bars + 2 * C::kStages, *qempty = qfull + 2, *qready = qfull + 4;
  uint64_t *pstored = qfull + 6, *pdone = qfull + 7;
  // [slot][b, first q head, rows, splits, first partial, counter index, last-arriver flag]: groups whose
  // partial this CTA has stored and whose arrival counter has yet to be looked at
  volatile int *pinfo = reinterpret_cast<volatile int *>(smem + C::kOffDesc) + 2 * kDescInts + 4;
  int *desc = reinterpret_cast<int *>(smem + C::kOffDesc);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // a kernel launched behind this one with programmatic stream serialisation may become resident now;
  // it blocks in griddepcontrol.wait until this grid has completed
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) {
    for (int i = 0; i < C::kStages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], C::kWarps);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&qfull[i], 1);
      mbar_init(&qempty[i], C::kWarps);
      mbar_init(&qready[i], 1);
    }
    mbar_init(pstored, C::kWarps);
    mbar_init(pdone, 1);
    fence_barrier_init();
  }
  __syncthreads();

  const PlanView pv = make_plan_view(p.plan_in_param ? pp.w : p.plan);
  const int total = pv.total_items;

  if (warp == C::kWarps) {
    // ======================= producer warp =======================
    if (lane == 0) {
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
    }
    // stage the per-sequence item offsets in shared memory (one coalesced fetch) so that decoding a
    // work item costs one global round trip instead of a chain of them
    int32_t *ib = reinterpret_cast<int32_t *>(smem + C::kOffItemBase);
    const bool ib_ok = pv.nseq + 1 <= C::kItemBaseCap;
    if (ib_ok) {
      for (int i = lane; i <= pv.nseq; i += 32) ib[i] = __ldg(pv.item_base + i);
      __syncwarp();
    }
    const int32_t *ibs = ib_ok ? ib : nullptr;
    // When launched with programmatic stream serialisation right behind the cache-scatter kernel, this
    // grid runs beside that kernel's tail.  What the scatter kernel writes -- the caches and the
    // scheduling words -- is touched only after griddepcontrol.wait (below, in front of the first cache
    // tile); the plan, the q rows and the block tables are inputs of the step that were complete before
    // the scatter kernel started, so the first item's decode, q load and table fetch overlap it too.
    bool synced = false;
    uint32_t st = 0, ph = 0;
    const int bs = p.block_size;
    const int bpt = kTile / bs;  // cache blocks per tile (divides 32)
    // Work items are handed out by a ticket (the list is longest-first): the first two items of a CTA
    // are fixed (its own index, and that plus the grid size), every further one comes from an atomic
    // counter in the workspace that is zero when the kernel starts.  Which CTA computes an item has no
    // influence on the item's bits.  The descriptor and the q rows of item i + 1 are published as soon as
    // the last tile of item i has been issued -- the consumers still have the tiles in the ring in
    // front of them -- so they are in shared memory (and, for an int8 cache, converted by the helper
    // warp) before the consumers ask for them.
    auto publish = [&](const WorkItem &w, int qs) {  // lane 0: descriptor + q rows into slot qs
      int *d = desc + qs * kDescInts;
      d[0] = w.b; d[1] = w.kvh; d[2] = w.row0; d[3] = w.nrows;
      d[4] = w.tok0; d[5] = w.tok1; d[6] = w.nsplit; d[7] = w.part;
      d[8] = w.grp; d[9] = w.part0; d[10] = w.qtok0; d[11] = w.ntok;
      // q rows of the item: for a decode batch one contiguous run (rows row0 .. row0 + nrows of the kv
      // head's group); for stacked query tokens the group's rows of every token, one run per token
      const uint32_t qbytes = (uint32_t)w.nrows * D * 2;
      mbar_arrive_expect_tx(&qfull[qs], qbytes);
      const uint32_t run = qbytes / (uint32_t)w.ntok;
      for (int tq = 0; tq < w.ntok; ++tq) {
        const char *qsrc = static_cast<const char *>(p.q) +
                           ((int64_t)(w.qtok0 + tq) * p.num_q_heads + w.kvh * p.group + w.row0) * (D * 2);
        bulk_load(smem + C::kOffQ + qs * C::kQSlotBytes + tq * run, qsrc, run, &qfull[qs]);
      }
    };
    int t_nxt = (int)blockIdx.x + (int)gridDim.x;  // the second item of a CTA is fixed too
    WorkItem w = decode_item(pv, blockIdx.x, p.num_kv_heads, p.group, C::kRows, ibs);  // grid <= items
    if (lane == 0) publish(w, 0);  // slot 0 is free at the start
    for (int qi = 0;; ++qi) {
      // the ticket of item qi + 1 is drawn here and used once this item's tiles are out: its latency
      // hides behind them, and a CTA never holds more than the item it loads (a ticket drawn any
      // earlier would pin one more item to this CTA and lengthen the tail of the grid by that item)
      int t_draw = 0;
      if (qi >= 1 && lane == 0) t_draw = 2 * (int)gridDim.x + (int)atomicAdd(p.sync, 1u);
      auto sync_once = [&]() {  // first item only: from here on the scatter kernel's writes are visible
        asm volatile("griddepcontrol.wait;" ::: "memory");
        synced = true;
      };
      const int ntok = w.tok1 - w.tok0;
      const int nblk_item = (ntok + bs - 1) / bs;
      const int32_t *trow = p.block_tables + (int64_t)w.b * p.max_blocks_per_seq + w.tok0 / bs;
      int tile = 0;
      for (int blk0 = 0; blk0 < nblk_item; blk0 += 32) {
        // 32 block ids per batch, one per lane; a batch holds whole tiles
        int my_id = 0;
        if (blk0 + lane < nblk_item) {
          my_id = __ldg(trow + blk0 + lane);
          if (my_id < 0 || my_id >= p.num_blocks) {
            report_status(p.status, p.epoch, kStatusOob);
            my_id = 0;  // stay inside the cache; the result of this item is undefined
          }
        }
        if (!synced) sync_once();
        const int nblk_batch = min(32, nblk_item - blk0);
        for (int jb = 0; jb < nblk_batch; jb += bpt, ++tile) {
          const int nv = min(kTile, ntok - tile * kTile);  // valid tokens of this tile
          const int nb_tile = (nv + bs - 1) / bs;
#pragma unroll 1
          for (int op = 0; op < 2; ++op) {
            if (!mbar_wait(&empty[st], ph ^ 1, kWaitLimit)) {
              report_status(p.status, p.epoch, kStatusTimeout);
              return;
            }
            uint8_t *dst = smem + st * C::kStageBytes;
            if (lane == 0) mbar_arrive_expect_tx(&full[st], (uint32_t)(nb_tile * bs * C::kRowBytes));
            for (int j = 0; j < nb_tile; ++j) {
              const int id = __shfl_sync(0xffffffffu, my_id, jb + j);
              if (lane == 0) {
                const CUtensorMap *tm = op == 0 ? &tm_k : &tm_v;
                // block-size-major cache: view [tokens][kv heads][head_dim], box {128 B, 1 head, block_size
                // tokens} at (x, head, first token of the block); head-major cache: view
                // [blocks x kv heads][block_size][head_dim], box {128 B, block_size tokens, 1} at
                // (x, 0, block x heads + head).  Either way the box lands as block_size rows of 128 bytes.
                const int y = p.cache_layout == 0 ? w.kvh : 0;
                const int z = p.cache_layout == 0 ? id * bs : id * p.num_kv_heads + w.kvh;
                // one 128-byte box per 64 elements (16-bit) / 128 elements (int8) of the head dimension;
                // x is a multiple of 64 elements = 128 bytes: TMA's 16-byte rule holds by construction
#pragma unroll
                for (int bx = 0; bx < C::kBoxes; ++bx)
                  tma_load_3d(dst + bx * (kTile * 128) + j * bs * 128, tm, bx * (KV8 ? 128 : 64), y, z, &full[st]);
              }
            }
            if (++st == C::kStages) { st = 0; ph ^= 1; }
          }
        }
      }
      if (!synced) sync_once();  // (an item without a tile cannot happen; the scheduling words need the wait)
      // item qi + 1 (or the end marker) into the other slot, once the consumers have let go of it
      if (qi >= 1) t_nxt = __shfl_sync(0xffffffffu, t_draw, 0);
      const int ns = (qi + 1) & 1;
      const uint32_t nph = ((qi + 1) >> 1) & 1;
      if (!mbar_wait(&qempty[ns], nph ^ 1, kWaitLimit)) {
        report_status(p.status, p.epoch, kStatusTimeout);
        return;
      }
      if (t_nxt >= total) {  // no work left: tell the consumers
        if (lane == 0) {
          desc[ns * kDescInts] = -1;
          mbar_arrive(&qfull[ns]);
        }
        break;
      }
      w = decode_item(pv, t_nxt, p.num_kv_heads, p.group, C::kRows, ibs);
      if (lane == 0) publish(w, ns);
    }
    return;
  }

  if (warp == C::kWarps + 1) {
    // ======================= arrival-counter warp =======================
    // Split partials are merged by the CTA that stores the LAST partial of a (sequence, kv head,
    // q-row block) group.  Finding that out takes a device-scope fence (the CTA's partial stores before
    // the counter) and an atomic on the group's counter: about two microseconds of latency that this
    // warp absorbs, so the consumer warps never wait for either.  The consumers announce a stored
    // partial on `pstored`, this warp answers on `pdone` with the flag in the group's slot.
    for (int k = 0;; ++k) {
      if (!mbar_wait(pstored, (uint32_t)(k & 1), kWaitLimit)) {
        report_status(p.status, p.epoch, kStatusTimeout);
        return;
      }
      volatile int *g = pinfo + (k & 3) * 8;
      if (g[0] < 0) return;  // the consumers are done
      if (lane == 0) {
        __threadfence();  // every consumer warp's partial stores (ordered before its arrival) precede the count
        const unsigned old = atomicAdd(p.sync + kSyncHeaderWords + g[5], 1u);
        __threadfence();  // ... and the other CTAs' partials precede whatever follows the answer
        g[6] = (old == (unsigned)(g[3] - 1)) ? 1 : 0;
        mbar_arrive(pdone);
      }
      __syncwarp();
    }
  }

  if (C::kAux && warp == C::kWarps + 2) {
    // ======================= Q-preparation warp (int8 KV) =======================
    // k_descale is folded into Q, and inside each 16-wide group of the head dimension the
    // contraction index is permuted so that the four bytes a lane gets from ldmatrix
    // (d = 16ks + 4q4 .. +3) are its two A registers.  This warp converts the rows of the NEXT item
    // while the consumers still work on the current one: word (row tile, k-step pair, lane,
    // 2 (ks & 1) + j) holds the fp16 pair Q[8nt + gid][16ks + 4q4 + 2j, + 1] * k_descale.
    for (int qi = 0;; ++qi) {
      const int qs = qi & 1;
      const uint32_t qph = (qi >> 1) & 1;
      if (!mbar_wait(&qfull[qs], qph, kWaitLimit)) {
        report_status(p.status, p.epoch, kStatusTimeout);
        return;
      }
      const int *dsc = desc + qs * kDescInts;
      const int b = dsc[0];
      if (b < 0) {
        if (lane == 0) mbar_arrive(&qready[qs]);
        return;
      }
      const int kvh = dsc[1], nrows = dsc[3];
      const T *qsm = reinterpret_cast<const T *>(smem + C::kOffQ + qs * C::kQSlotBytes);
      uint32_t *qfrag = reinterpret_cast<uint32_t *>(smem + C::kOffQFrag + qs * C::kQFragBytes);
      float *score_shift = reinterpret_cast<float *>(smem + C::kOffQFrag + qs * C::kQFragBytes + NT * 4 * 32 * 16);
      const float *ksc = p.k_descale + kvh * D;
      for (int u = lane; u < C::kRows * 64; u += 32) {
        const int r = u >> 6, dp = u & 63;  // q row, index of the pair of head-dim columns
        float e0 = 0.f, e1 = 0.f;
        if (r < nrows) {
          const float2 sc = __ldg(reinterpret_cast<const float2 *>(ksc + 2 * dp));
          e0 = to_f32<T>(qsm[r * D + 2 * dp]) * sc.x;
          e1 = to_f32<T>(qsm[r * D + 2 * dp + 1]) * sc.y;
        }
        const int ks = dp >> 3, qq = (dp >> 1) & 3, j = dp & 1;
        const uint32_t packed = pack2<__half>(e0, e1);
        qfrag[(((r >> 3) * 4 + (ks >> 1)) * 32 + (r & 7) * 4 + qq) * 4 + 2 * (ks & 1) + j] = packed;
        if (p.lse != nullptr) {
          // the K bytes enter the MMA as k + 1152 instead of k + k_offset: every score of q row r is
          // too large by sum_d Q~[r][d] (1152 - k_offset[d]).  The softmax does not see that, the
          // log-sum-exp does: the warp (32 column pairs of one row) adds up its half of the sum.
          const __half2 h2 = *reinterpret_cast<const __half2 *>(&packed);
          float o0 = 1152.f, o1 = 1152.f;
          if (p.k_offset != nullptr) {
            o0 -= (float)__ldg(p.k_offset + kvh * D + 2 * dp);
            o1 -= (float)__ldg(p.k_offset + kvh * D + 2 * dp + 1);
          }
          float part = fmaf(__low2float(h2), o0, __high2float(h2) * o1);
#pragma unroll
          for (int sh = 16; sh > 0; sh >>= 1) part += __shfl_xor_sync(0xffffffffu, part, sh);
          if (lane == 0) score_shift[2 * r + (dp >> 5)] = part;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&qready[qs]);  // release: the fragments are visible to whoever waits
    }
  }

  // ======================= consumer warps =======================
  const int gid = lane >> 2, q4 = lane & 3;
  const int t0 = warp * 16 * SUBS;           // this warp's token rows inside a tile
  const int mat = lane >> 3, mr = lane & 7;  // ldmatrix: matrix id and row supplied by this lane
  const uint32_t stage0 = smem_u32(smem);
  // byte offsets of the ldmatrix rows this lane supplies (swizzle: 16-byte chunk ^= row & 7)
  //   K 16-bit, K int8, V int8: matrices 1,3 are the tokens +8;  V 16-bit: matrices 2,3
  const uint32_t row_m1 = (uint32_t)(t0 + (mat & 1) * 8 + mr) * 128u;
  const uint32_t row_m2 = (uint32_t)(t0 + (mat >> 1) * 8 + mr) * 128u;
  const int tid = threadIdx.x;

  uint32_t st = 0, ph = 0;
  // Merge of split partials.  When an item of a multi-split group has stored its partial, the warps
  // announce it to the arrival-counter warp; at the next item's barrier they pick up the answer and, if
  // this CTA stored the group's last partial, all warps merge the group (in split order).
  int n_stored = 0, n_checked = 0;  // groups announced / answers picked up (uniform)
  auto merge_if_last = [&]() -> bool {  // run by all consumer threads, after a barrier
    if (n_checked == n_stored) return true;
    if (!mbar_wait(pdone, (uint32_t)(n_checked & 1), kWaitLimit)) return false;
    const volatile int *g = pinfo + (n_checked & 3) * 8;
    if (g[6]) {
      const int gq0 = g[0], ghq0 = g[1], gnrows = g[2], gns = g[3], gpart0 = g[4], gntok = g[7];
      const int gt = gntok > 1 ? p.group : 16;  // q rows per stacked token (a decode item is one token)
      for (int r = warp; r < gnrows; r += C::kWarps) {
        const int tq = r / gt, j = r - tq * gt;
        merge_row<T, D>(p, (int64_t)(gq0 + tq) * p.num_q_heads + ghq0 + j, ghq0 + j, gns, gpart0 + tq * gns, lane);
      }
    }
    ++n_checked;
    return true;
  };

  for (int qi = 0;; ++qi) {
    const int qs = qi & 1;
    const uint32_t qph = (qi >> 1) & 1;
    if (!mbar_wait(KV8 ? &qready[qs] : &qfull[qs], qph, kWaitLimit)) {
      report_status(p.status, p.epoch, kStatusTimeout);
      return;
    }
    const int *dsc = desc + qs * kDescInts;
    const int b = dsc[0];
    if (b < 0) break;  // the producer found no further work item
    const int kvh = dsc[1], row0 = dsc[2], nrows = dsc[3];
    const int tok0 = dsc[4], tok1 = dsc[5], nsplit = dsc[6], part = dsc[7];
    const int grp = dsc[8], part0 = dsc[9], qtok0 = dsc[10], ntok = dsc[11];
    const int gt = ntok > 1 ? p.group : 16;  // q rows per stacked query token: row r belongs to token r / gt
    // additive mask: element offset of context token tok0 in the mask row of each of this lane's q rows
    // (rows 8nt + 2q4 + j), once per item; -1 for rows the item does not have
    int64_t mrow[MASK ? NT : 1][2];
    if (MASK) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int r = 8 * nt + 2 * q4 + j;
          mrow[nt][j] = -1;
          if (r < nrows) {
            const int tq = r / gt;
            mrow[nt][j] = (int64_t)(qtok0 + tq) * p.mask_batch_stride +
                          (int64_t)(kvh * p.group + row0 + r - tq * gt) * p.mask_head_stride + tok0;
          }
        }
    }
    float *mbuf = reinterpret_cast<float *>(smem + C::kOffMerge + (C::kMergeBufs == 2 ? (qi & 1) * C::kMergeBytes : 0));
    float2 *mlbuf = reinterpret_cast<float2 *>(smem + C::kOffMl + (C::kMergeBufs == 2 ? (qi & 1) * C::kMlBytes : 0));

    // ---- Q^T fragments (B operand): lane holds q row 8nt + gid, rows >= nrows are zero ----
    uint32_t qb[kKS][NT][2];
    {
      if (!KV8) {
        const T *qsm = reinterpret_cast<const T *>(smem + C::kOffQ + qs * C::kQSlotBytes);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const bool valid = 8 * nt + gid < nrows;
          const T *qr = qsm + (8 * nt + gid) * D;
#pragma unroll
          for (int ks = 0; ks < kKS; ++ks) {
            const int c = 16 * ks + 2 * q4;
            qb[ks][nt][0] = valid ? *reinterpret_cast<const uint32_t *>(qr + c) : 0u;
            qb[ks][nt][1] = valid ? *reinterpret_cast<const uint32_t *>(qr + c + 8) : 0u;
          }
        }
      } else {
        const uint32_t *qfrag = reinterpret_cast<const uint32_t *>(smem + C::kOffQFrag + qs * C::kQFragBytes);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int kp = 0; kp < 4; ++kp) {
            const uint4 v = *reinterpret_cast<const uint4 *>(qfrag + ((nt * 4 + kp) * 32 + lane) * 4);
            qb[2 * kp][nt][0] = v.x; qb[2 * kp][nt][1] = v.y;
            qb[2 * kp + 1][nt][0] = v.z; qb[2 * kp + 1][nt][1] = v.w;
          }
      }
    }
    // int8 KV with the lse output: the partial score offsets of the lse correction are needed at the merge
    // below; warp 0 takes a copy so that the slot can be handed back right away
    float *shift_copy = reinterpret_cast<float *>(smem + C::kOffShift) + (qi & 1) * 32;
    if (KV8 && p.lse != nullptr && tid < 2 * C::kRows)
      shift_copy[tid] = reinterpret_cast<const float *>(smem + C::kOffQFrag + qs * C::kQFragBytes + NT * 4 * 32 * 16)[tid];
    __syncwarp();
    if (lane == 0) mbar_arrive(&qempty[qs]);

    // running state of this lane's two q rows per row tile (rows 8nt + 2q4, + 1)
    // The row sums l come from the tensor cores too: a tile of ones in place of V^T gives
    // sum_tokens P (of exactly the rounded probabilities the output is built from) in ol[nt][0..1].
    float m_run[NT][2];
    float ol[NT][4];
    float o[kKS][NT][4];  // O^T: [16-wide slice of head_dim][row tile]
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      m_run[nt][0] = m_run[nt][1] = kNeg;
      ol[nt][0] = ol[nt][1] = ol[nt][2] = ol[nt][3] = 0.f;
    }
#pragma unroll
    for (int mt = 0; mt < kKS; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) o[mt][nt][0] = o[mt][nt][1] = o[mt][nt][2] = o[mt][nt][3] = 0.f;

    const int ntiles = (tok1 - tok0 + kTile - 1) / kTile;
    for (int ti = 0; ti < ntiles; ++ti) {
      const int nv = min(kTile, tok1 - tok0 - ti * kTile);
      const bool active = t0 < nv;  // warp-uniform: any of this warp's tokens valid
      // ---------------- S^T = K Q^T ----------------
      float s[SUBS][NT][4];
#pragma unroll
      for (int sb = 0; sb < SUBS; ++sb)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) s[sb][nt][0] = s[sb][nt][1] = s[sb][nt][2] = s[sb][nt][3] = 0.f;
      // additive mask of this lane's (token, row) pairs, fetched before the tile is waited for;
      // same element order as s[sb][nt][0..3]
      float mk[SUBS][NT][4];
      if (MASK) {
#pragma unroll
        for (int sb = 0; sb < SUBS; ++sb)
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            mk[sb][nt][0] = mk[sb][nt][1] = mk[sb][nt][2] = mk[sb][nt][3] = 0.f;
            if (active) {
              const int tw = t0 + 16 * sb + gid;  // token inside the tile
              const int tk = ti * kTile + tw;     // ... and inside the item
#pragma unroll
              for (int j = 0; j < 2; ++j) {
                const int64_t base = mrow[MASK ? nt : 0][j];
                if (base >= 0) {
                  if (tw < nv) mk[sb][nt][j] = load_mask_elem(p.mask, p.mask_dtype, base + tk);
                  if (tw + 8 < nv) mk[sb][nt][2 + j] = load_mask_elem(p.mask, p.mask_dtype, base + tk + 8);
                }
              }
            }
          }
      }
      if (!mbar_wait(&full[st], ph, kWaitLimit)) {
        report_status(p.status, p.epoch, kStatusTimeout);
        return;
      }
      if (active) {
#pragma unroll
        for (int sb = 0; sb < SUBS; ++sb) {
          if (SUBS > 1 && t0 + 16 * sb >= nv) break;  // warp-uniform
          const uint32_t kbase = stage0 + st * C::kStageBytes + row_m1 + (uint32_t)sb * (16u * 128u);
          if (!KV8) {
#pragma unroll
            for (int ks = 0; ks < kKS; ++ks) {
              const uint32_t cc = (uint32_t)(2 * (ks & 3) + (mat >> 1));
              const uint32_t addr = kbase + (uint32_t)(ks >> 2) * (kTile * 128) + ((cc ^ (uint32_t)mr) << 4);
              uint32_t a0, a1, a2, a3;
              ldmatrix_x4(addr, a0, a1, a2, a3);
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) mma16816<MT>(s[sb][nt], a0, a1, a2, a3, qb[ks][nt][0], qb[ks][nt][1]);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t cc = (uint32_t)(2 * i + (mat >> 1));
              uint32_t r0, r1, r2, r3;  // (tokens lo, 2i) (tokens hi, 2i) (lo, 2i+1) (hi, 2i+1)
              ldmatrix_x4(kbase + ((cc ^ (uint32_t)mr) << 4), r0, r1, r2, r3);
              r0 ^= 0x80808080u; r1 ^= 0x80808080u; r2 ^= 0x80808080u; r3 ^= 0x80808080u;
              {
                const uint32_t a0 = bytes_to_half2_biased(r0, 0x5140u), a1 = bytes_to_half2_biased(r1, 0x5140u);
                const uint32_t a2 = bytes_to_half2_biased(r0, 0x5342u), a3 = bytes_to_half2_biased(r1, 0x5342u);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                  mma16816<MT>(s[sb][nt], a0, a1, a2, a3, qb[2 * i][nt][0], qb[2 * i][nt][1]);
              }
              {
                const uint32_t a0 = bytes_to_half2_biased(r2, 0x5140u), a1 = bytes_to_half2_biased(r3, 0x5140u);
                const uint32_t a2 = bytes_to_half2_biased(r2, 0x5342u), a3 = bytes_to_half2_biased(r3, 0x5342u);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                  mma16816<MT>(s[sb][nt], a0, a1, a2, a3, qb[2 * i + 1][nt][0], qb[2 * i + 1][nt][1]);
              }
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[st]);
      if (++st == C::kStages) { st = 0; ph ^= 1; }

      // ---------------- online softmax ----------------
      // s[sb][nt]: [0] (token gid, row 2q4) [1] (token gid, row 2q4+1) [2] (token gid+8, row 2q4) [3] (gid+8, 2q4+1)
      uint32_t pb[SUBS][NT][2];
      if (active) {
        const float c = p.scale_log2e;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          float x[SUBS][4];
          float mx0 = kNeg, mx1 = kNeg;
#pragma unroll
          for (int sb = 0; sb < SUBS; ++sb) {
            const int tw = t0 + 16 * sb + gid;
            const bool dead_lo = tw >= nv, dead_hi = tw + 8 >= nv;  // past the end of the range
            x[sb][0] = s[sb][nt][0] * c; x[sb][1] = s[sb][nt][1] * c;
            x[sb][2] = s[sb][nt][2] * c; x[sb][3] = s[sb][nt][3] * c;
            if (MASK) {
              const float l2e = 1.4426950408889634f;
              x[sb][0] = fmaf(mk[sb][nt][0], l2e, x[sb][0]); x[sb][1] = fmaf(mk[sb][nt][1], l2e, x[sb][1]);
              x[sb][2] = fmaf(mk[sb][nt][2], l2e, x[sb][2]); x[sb][3] = fmaf(mk[sb][nt][3], l2e, x[sb][3]);
            }
            if (dead_lo) x[sb][0] = x[sb][1] = kNeg;
            if (dead_hi) x[sb][2] = x[sb][3] = kNeg;
            mx0 = fmaxf(mx0, fmaxf(x[sb][0], x[sb][2]));
            mx1 = fmaxf(mx1, fmaxf(x[sb][1], x[sb][3]));
          }
#pragma unroll
          for (int sh = 4; sh <= 16; sh <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, sh));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, sh));
          }
          const float mn0 = fmaxf(m_run[nt][0], mx0), mn1 = fmaxf(m_run[nt][1], mx1);
          const float al0 = fast_exp2(m_run[nt][0] - mn0), al1 = fast_exp2(m_run[nt][1] - mn1);
          m_run[nt][0] = mn0;
          m_run[nt][1] = mn1;
          if (al0 != 1.f || al1 != 1.f) {
            ol[nt][0] *= al0; ol[nt][1] *= al1;
#pragma unroll
            for (int mt = 0; mt < kKS; ++mt) {
              o[mt][nt][0] *= al0; o[mt][nt][2] *= al0;
              o[mt][nt][1] *= al1; o[mt][nt][3] *= al1;
            }
          }
#pragma unroll
          for (int sb = 0; sb < SUBS; ++sb) {
            const float e0 = fast_exp2(x[sb][0] - mn0), e2 = fast_exp2(x[sb][2] - mn0);
            const float e1 = fast_exp2(x[sb][1] - mn1), e3 = fast_exp2(x[sb][3] - mn1);
            // probabilities (token-major) -> P^T fragments: (tokens 2q4, 2q4+1 | +8; row gid)
            pb[sb][nt][0] = movmatrix_trans(pack2<MT>(e0, e1));
            pb[sb][nt][1] = movmatrix_trans(pack2<MT>(e2, e3));
          }
        }
      }

      // ---------------- O^T += V^T P^T ----------------
      if (!mbar_wait(&full[st], ph, kWaitLimit)) {
        report_status(p.status, p.epoch, kStatusTimeout);
        return;
      }
      if (active) {
        uint8_t *vst = smem + st * C::kStageBytes;
        if (nv < t0 + 16 * SUBS) {
          // rows past the end of the range may hold anything (also NaN): zero them so that
          // 0 * garbage cannot reach the accumulators
          constexpr int kChunks = C::kRowBytes / 16;
          for (int idx = lane; idx < 16 * SUBS * kChunks; idx += 32) {
            const int r = idx / kChunks, ch = idx - r * kChunks;
            if (t0 + r >= nv) {
              uint8_t *dst = vst + (ch >> 3) * (kTile * 128) + (t0 + r) * 128 + (ch & 7) * 16;
              *reinterpret_cast<uint4 *>(dst) = make_uint4(0u, 0u, 0u, 0u);
            }
          }
          fence_proxy_async();
          __syncwarp();
        }
#pragma unroll
        for (int sb = 0; sb < SUBS; ++sb) {
          if (SUBS > 1 && t0 + 16 * sb >= nv) break;  // warp-uniform
          {
            const uint32_t ones = std::is_same<MT, __half>::value ? 0x3C003C00u : 0x3F803F80u;  // 1.0 twice
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
              mma16816<MT>(ol[nt], ones, ones, ones, ones, pb[sb][nt][0], pb[sb][nt][1]);
          }
          if (!KV8) {
            const uint32_t vbase = stage0 + st * C::kStageBytes + row_m2 + (uint32_t)sb * (16u * 128u);
#pragma unroll
            for (int mt = 0; mt < kKS; ++mt) {
              const uint32_t cc = (uint32_t)(2 * (mt & 3) + (mat & 1));
              const uint32_t addr = vbase + (uint32_t)(mt >> 2) * (kTile * 128) + ((cc ^ (uint32_t)mr) << 4);
              uint32_t a0, a1, a2, a3;  // (d lo, tok lo) (d hi, tok lo) (d lo, tok hi) (d hi, tok hi)
              ldmatrix_x4_trans(addr, a0, a1, a2, a3);
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) mma16816<MT>(o[mt][nt], a0, a1, a2, a3, pb[sb][nt][0], pb[sb][nt][1]);
            }
          } else {
            const uint32_t vbase = stage0 + st * C::kStageBytes + row_m1 + (uint32_t)sb * (16u * 128u);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t cc = (uint32_t)(2 * i + (mat >> 1));
              uint32_t r0, r1, r2, r3;  // (tok lo, 2i) (tok hi, 2i) (tok lo, 2i+1) (tok hi, 2i+1)
              ldmatrix_x4_trans(vbase + ((cc ^ (uint32_t)mr) << 4), r0, r1, r2, r3);
              r0 ^= 0x80808080u; r1 ^= 0x80808080u; r2 ^= 0x80808080u; r3 ^= 0x80808080u;
              // bytes 0,2: head-dim column 16c + 2 gid (tile rows 0..7); bytes 1,3: column + 1 (rows 8..15)
              {
                const uint32_t a0 = bytes_to_half2_biased(r0, 0x5240u), a1 = bytes_to_half2_biased(r0, 0x5341u);
                const uint32_t a2 = bytes_to_half2_biased(r1, 0x5240u), a3 = bytes_to_half2_biased(r1, 0x5341u);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                  mma16816<MT>(o[2 * i][nt], a0, a1, a2, a3, pb[sb][nt][0], pb[sb][nt][1]);
              }
              {
                const uint32_t a0 = bytes_to_half2_biased(r2, 0x5240u), a1 = bytes_to_half2_biased(r2, 0x5341u);
                const uint32_t a2 = bytes_to_half2_biased(r3, 0x5240u), a3 = bytes_to_half2_biased(r3, 0x5341u);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                  mma16816<MT>(o[2 * i + 1][nt], a0, a1, a2, a3, pb[sb][nt][0], pb[sb][nt][1]);
              }
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[st]);
      if (++st == C::kStages) { st = 0; ph ^= 1; }
    }

    // ---------------- merge the warps' states ----------------
    // Every warp publishes (m, l) of its rows and its un-scaled O^T; after one barrier each
    // output element is reduced over the warps with the weights 2^(m_w - M).
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int r0 = 8 * nt + 2 * q4;
      if (gid == 0) {
        mlbuf[warp * 16 + r0] = make_float2(m_run[nt][0], ol[nt][0]);
        mlbuf[warp * 16 + r0 + 1] = make_float2(m_run[nt][1], ol[nt][1]);
      }
      float *w0 = mbuf + (warp * C::kRows + r0) * C::kMergeStride, *w1 = w0 + C::kMergeStride;
#pragma unroll
      for (int mt = 0; mt < kKS; ++mt) {
        // accumulator columns: 16-bit KV  d = 16mt + gid, + 8;  int8 KV  d = 16mt + 2 gid, + 1
        const int da = KV8 ? 16 * mt + 2 * gid : 16 * mt + gid;
        const int db = KV8 ? da + 1 : da + 8;
        w0[da] = o[mt][nt][0]; w1[da] = o[mt][nt][1];
        w0[db] = o[mt][nt][2]; w1[db] = o[mt][nt][3];
      }
    }
    named_bar_sync(1, C::kConsumerThreads);
    if (!merge_if_last()) {
      report_status(p.status, p.epoch, kStatusTimeout);
      return;
    }
    for (int u = tid; u < C::kRows * (D / 4); u += C::kConsumerThreads) {
      const int row = u / (D / 4), c4 = (u - row * (D / 4)) * 4;  // four consecutive head-dim columns of one row
      if (row < nrows) {
        float2 ml[C::kWarps];
        float M = kNeg;
#pragma unroll
        for (int w2 = 0; w2 < C::kWarps; ++w2) {
          ml[w2] = mlbuf[w2 * 16 + row];
          M = fmaxf(M, ml[w2].x);
        }
        float L = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w2 = 0; w2 < C::kWarps; ++w2) {
          const float f = fast_exp2(ml[w2].x - M);
          L = fmaf(ml[w2].y, f, L);
          const float4 v = *reinterpret_cast<const float4 *>(mbuf + (w2 * C::kRows + row) * C::kMergeStride + c4);
          acc.x = fmaf(v.x, f, acc.x); acc.y = fmaf(v.y, f, acc.y);
          acc.z = fmaf(v.z, f, acc.z); acc.w = fmaf(v.w, f, acc.w);
        }
        if (KV8) {  // remove the bias the V bytes carried: sum_t p (v + 1152) = O + 1152 l
          acc.x = fmaf(-1152.f, L, acc.x); acc.y = fmaf(-1152.f, L, acc.y);
          acc.z = fmaf(-1152.f, L, acc.z); acc.w = fmaf(-1152.f, L, acc.w);
        }
        const int tq = row / gt;
        const int hq = kvh * p.group + row0 + row - tq * gt;
        const int64_t orow = (int64_t)(qtok0 + tq) * p.num_q_heads + hq;  // row of query / out / lse
        if (p.lse != nullptr) {
          if (KV8)  // back to the scores of the true K values (see the Q preparation)
            M -= (shift_copy[2 * row] + shift_copy[2 * row + 1]) * p.scale_log2e;
          if (nsplit == 1 && c4 == 0) p.lse[orow] = (M + log2f(L)) * kLn2;
        }
        if (nsplit == 1) {
          const float inv = 1.f / L;
          float r0 = acc.x * inv, r1 = acc.y * inv, r2 = acc.z * inv, r3 = acc.w * inv;
          if (KV8) {
            const float4 vs = __ldg(reinterpret_cast<const float4 *>(p.v_descale + kvh * D + c4));
            if (p.v_offset != nullptr) {
              const int4 vo = __ldg(reinterpret_cast<const int4 *>(p.v_offset + kvh * D + c4));
              r0 += (float)vo.x; r1 += (float)vo.y; r2 += (float)vo.z; r3 += (float)vo.w;
            }
            r0 *= vs.x; r1 *= vs.y; r2 *= vs.z; r3 *= vs.w;
          }
          uint2 pk;
          pk.x = pack2<T>(r0, r1);
          pk.y = pack2<T>(r2, r3);
          *reinterpret_cast<uint2 *>(static_cast<T *>(p.out) + orow * D + c4) = pk;
        } else {
          const int64_t prow = (int64_t)(part + tq * nsplit) * p.num_q_heads + hq;
          *reinterpret_cast<float4 *>(p.part_o + prow * D + c4) = acc;
          if (c4 == 0) *reinterpret_cast<float2 *>(p.part_ml + prow * 2) = make_float2(M, L);
        }
      }
    }
    if (nsplit > 1 && p.fused_merge != 0) {
      if (tid == 0) {
        volatile int *g = pinfo + (n_stored & 3) * 8;
        g[0] = qtok0; g[1] = kvh * p.group + row0; g[2] = nrows; g[3] = nsplit; g[4] = part0; g[5] = grp;
        g[7] = ntok;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(pstored);  // release: this warp's partial stores are ordered before it
      ++n_stored;
    }
    if (C::kMergeBufs == 1) named_bar_sync(1, C::kConsumerThreads);  // the merge buffer is reused by the next item
  }
  // the last group this CTA stored, then the arrival-counter warp is told to leave
  const bool ok = merge_if_last();
  if (tid == 0) pinfo[(n_stored & 3) * 8] = -1;
  __syncwarp();
  if (lane == 0) mbar_arrive(pstored);
  if (!ok) report_status(p.status, p.epoch, kStatusTimeout);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// View of one cache as [tokens = num_blocks * block_size][kv heads][head_dim]; a box is one head's
// rows of one cache block (block_size tokens) and 128 bytes of the head dimension.
int make_cache_tmap(CUtensorMap *tm, const void *cache, const MscoPaDesc &d) {
  const int kD = d.head_dim;
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return fail(MSCO_ERR_CUDA, "paged_attention: cuTensorMapEncodeTiled is not available");
  const bool kv8 = d.kv_dtype == MSCO_DTYPE_I8;
  const int es = kv8 ? 1 : 2;
  const bool head_major = d.cache_layout == 1;
  const cuuint64_t dims[3] = {(cuuint64_t)kD, head_major ? (cuuint64_t)d.block_size : (cuuint64_t)d.num_kv_heads,
                              head_major ? (cuuint64_t)d.num_blocks * (cuuint64_t)d.num_kv_heads
                                         : (cuuint64_t)d.num_blocks * (cuuint64_t)d.block_size};
  const cuuint64_t strides[2] = {(cuuint64_t)kD * es, head_major ? (cuuint64_t)d.block_size * kD * es
                                                                 : (cuuint64_t)d.num_kv_heads * kD * es};
  const cuuint32_t box[3] = {(cuuint32_t)(kv8 ? 128 : 64), head_major ? (cuuint32_t)d.block_size : 1u,
                             head_major ? 1u : (cuuint32_t)d.block_size};
  const cuuint32_t estr[3] = {1u, 1u, 1u};
  const CUtensorMapDataType dt = kv8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                     : (d.kv_dtype == MSCO_DTYPE_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                                     : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
  const CUresult r = enc(tm, dt, 3, const_cast<void *>(cache), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MSCO_ERR_CUDA, "paged_attention: cuTensorMapEncodeTiled failed (%d)", (int)r);
  return MSCO_OK;
}

template <typename T, int D, bool KV8, int NT, bool MASK, int SUBS, int PW>
int launch_sized(const MscoPaPlan *plan, const PaParams &p, const PlanParamT<PW> &pp, const CUtensorMap &tk,
                 const CUtensorMap &tv, cudaStream_t stream, bool after_kernel) {
  using C = Cfg<D, KV8, NT, SUBS>;
  static_assert(C::kDynSmem <= 232448, "shared memory budget of one SM exceeded");
  auto kfn = pa_tma_kernel<T, D, KV8, NT, MASK, SUBS, PW>;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [&] {
    attr_err = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kDynSmem);
  });
  if (attr_err != cudaSuccess)
    return fail(MSCO_ERR_CUDA, "paged_attention: cudaFuncSetAttribute failed: %s", cudaGetErrorString(attr_err));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(plan->grid);
  cfg.blockDim = dim3(C::kThreads);
  cfg.dynamicSmemBytes = C::kDynSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = after_kernel ? 1 : 0;
  MSCO_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kfn, tk, tv, p, pp));
  return MSCO_OK;
}

// Small plans of the unmasked variants (the decode hot path) take the small parameter form.
template <typename T, int D, bool KV8, int NT, bool MASK, int SUBS>
int launch_one(const MscoPaPlan *plan, const PaParams &p, const PlanParam &pp, const CUtensorMap &tk,
               const CUtensorMap &tv, cudaStream_t stream, bool after_kernel) {
  if (!MASK && p.plan_in_param && plan->plan_words <= (size_t)kPlanParamWordsSmall)
    return launch_sized<T, D, KV8, NT, false, SUBS, kPlanParamWordsSmall>(
        plan, p, *reinterpret_cast<const PlanParamSmall *>(&pp), tk, tv, stream, after_kernel);
  return launch_sized<T, D, KV8, NT, MASK, SUBS, kPlanParamWords>(plan, p, pp, tk, tv, stream, after_kernel);
}

}  // namespace

// Tokens per tile of the kernel variant that serves `d`: a tile holds whole cache blocks.
static int tile_tokens(const MscoPaDesc &d) {
  if (d.head_dim == 256) return 64;
  if ((d.kv_dtype == MSCO_DTYPE_I8 || d.head_dim == 64) && d.num_q_heads / d.num_kv_heads <= 8) return 256;
  return 128;
}

bool pa_tma_supported(const MscoPaDesc &d) {
  const int bs = d.block_size;
  const bool bs_ok = (bs == 16 || bs == 32 || bs == 64 || bs == 128) && bs <= tile_tokens(d);
  const bool kv8 = d.kv_dtype == MSCO_DTYPE_I8;
  const bool d_ok = d.head_dim == 128 || (!kv8 && (d.head_dim == 64 || d.head_dim == 256));
  return d_ok && bs_ok && d.num_blocks * (int64_t)bs < (1ll << 31) &&
         d.num_blocks * (int64_t)d.num_kv_heads < (1ll << 31);
}

int pa_tma_rows_per_item(const MscoPaDesc &d) {
  const int g = d.num_q_heads / d.num_kv_heads;
  return (g > 8 && d.head_dim != 256) ? 16 : 8;
}

int launch_pa_tma(const MscoPaPlan *plan, const PaParams &p, const PlanParam &pp, cudaStream_t stream,
                  bool after_kernel) {
  if (plan->total_items == 0) return MSCO_OK;
  if ((reinterpret_cast<uintptr_t>(p.q) & 15) || (reinterpret_cast<uintptr_t>(p.key_cache) & 15) ||
      (reinterpret_cast<uintptr_t>(p.value_cache) & 15) || (reinterpret_cast<uintptr_t>(p.out) & 7))
    return fail(MSCO_ERR_INVALID_ARG, "paged_attention: query / caches must be 16-byte aligned");
  CUtensorMap tk, tv;
  {
    std::lock_guard<std::mutex> g(plan->tm_mutex);
    if (plan->tm_k_ptr != p.key_cache) {
      int rc = make_cache_tmap(reinterpret_cast<CUtensorMap *>(plan->tm_k), p.key_cache, plan->desc);
      if (rc != MSCO_OK) return rc;
      plan->tm_k_ptr = p.key_cache;
    }
    if (plan->tm_v_ptr != p.value_cache) {
      int rc = make_cache_tmap(reinterpret_cast<CUtensorMap *>(plan->tm_v), p.value_cache, plan->desc);
      if (rc != MSCO_OK) return rc;
      plan->tm_v_ptr = p.value_cache;
    }
    tk = *reinterpret_cast<const CUtensorMap *>(plan->tm_k);
    tv = *reinterpret_cast<const CUtensorMap *>(plan->tm_v);
  }
  const bool kv8 = plan->desc.kv_dtype == MSCO_DTYPE_I8;
  const bool g16 = plan->rows_per_item == 16;
  const bool f16 = plan->desc.q_dtype == MSCO_DTYPE_F16;
  const bool masked = plan->desc.mask_type != 0;
  const int hd = plan->desc.head_dim;
#define MSCO_GO(T, D, A, B, S)                                                                      \
  do {                                                                                              \
    if (masked) return launch_one<T, D, A, B, true, S>(plan, p, pp, tk, tv, stream, after_kernel);  \
    return launch_one<T, D, A, B, false, S>(plan, p, pp, tk, tv, stream, after_kernel);             \
  } while (0)
#define MSCO_GO_T(T)                                                      \
  do {                                                                    \
    if (hd == 64) { if (g16) MSCO_GO(T, 64, false, 2, 1); else MSCO_GO(T, 64, false, 1, 2); } \
    if (hd == 256) MSCO_GO(T, 256, false, 1, 1);                          \
    if (kv8) {                                                            \
      if (g16) MSCO_GO(T, 128, true, 2, 1);                               \
      MSCO_GO(T, 128, true, 1, 2);                                        \
    }                                                                     \
    if (g16) MSCO_GO(T, 128, false, 2, 1);                                \
    MSCO_GO(T, 128, false, 1, 1);                                         \
  } while (0)
  if (f16) MSCO_GO_T(__half);
  MSCO_GO_T(__nv_bfloat16);
#undef MSCO_GO_T
#undef MSCO_GO
}

}  // namespace msco

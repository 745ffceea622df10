// Bidirectional varlen attention over the slot-mapped paged cache for requests with many
// query rows (prefill, refresh), tcgen05 + TMEM, bf16/fp16, head_dim 64/128.
//
// One CTA = one (request, KV head, tile of 256 virtual rows); a virtual row is a (query,
// head-of-the-GQA-group) pair.  The 256 rows are two row blocks of 128 that share every staged
// K/V tile: a tile of 64 keys is gathered once per 256 rows instead of once per 128 as in the
// kernel that gives every 128 rows a CTA of their own (attention_tc.cu).  One CTA per SM, roles
// that hand over through mbarriers only:
//   warps 0-7   own the rows: thread t owns virtual row t of the tile (row block t / 128, TMEM
//               lane t % 128): tcgen05.ld of its scores, online softmax in the exp2 domain, the
//               weights P written back to TMEM over the scores they came from (two per 32-bit
//               column), where the P V product reads them as its A operand.  They do nothing
//               else in the loop;
//   warps 8,9   one thread each issues the tensor-core products of one row block: S(i+1) = Q K(i+1)^T
//               one tile ahead of the softmax into one of two S buffers, and O += P(i) V(i);
//   warps 10,11 gather the K tiles (16-byte cp.async into the 128-byte-swizzled operand layout,
//               3 stages), look up the slot map and publish which keys of a tile take no part;
//   warps 12,13 gather the V tiles (2 stages).
// TMEM: 512 columns; row block r holds S buffers at columns 256 r and 256 r + 64 (P(i) takes the
// first 32 columns of S buffer i & 1) and O at 256 r + 128.  Shared memory: Q (2 blocks), K (3
// stages), V (2 stages).
//   bar_k[s]    K stage s has landed           bar_v[s]     V stage s has landed
//   bar_s[r][b] S buffer b of block r is done  bar_p[r][b]  P is written over S buffer b of block r
//   bar_o[r][i & 1]  P V(i) of block r is done bar_q[r]     the query tile of block r is in place
// (one arrival per warp: its lanes synchronise, one lane arrives; the product barriers are
// tcgen05.commit arrivals).
// The softmax of a row block never waits for its own P V product: P(i) lives in the S buffer it
// was computed from (S(i+2) is issued after P V(i) by the same thread, and the tensor cores keep
// that order), and O, which the products accumulate in place, is only touched by the threads when
// a row's reference maximum moves, which then (and only then) waits for P V(i-1).
// A K stage is refilled when the S products of BOTH row blocks that read it are done, a V stage
// when both P V products are; only the loader warps look at both blocks' barriers, so the two
// blocks need not run in step.  A parity wait is only right while the barrier is at most one
// phase past the awaited one: every product that completes a later phase needs something the
// waiting thread provides after its wait (which is why the P and P V barriers alternate with the
// tile's parity).
//
// PAIR (requests of at least 1024 virtual rows, head_dim 128): two CTAs of a cluster, 512 rows,
// work as one.  Every product is a tcgen05.mma.cta_group::2 over row block r of BOTH CTAs (M =
// 256), issued by the first CTA's issuing threads: half the tensor-core instructions per row,
// which is what bounds the single-CTA form (one thread retires a product per ~100 cycles
// whatever its size).  The B operand is split between the CTAs: each gathers 32 of a tile's 64
// keys (K) and 64 of the 128 head dimensions of every key (V), so a tile crosses L2 -> shared
// memory once per 512 rows.  The barriers the issuing threads wait on live in the first CTA and
// take arrivals from both; the product barriers exist in both CTAs and the commits arrive on
// both.  No load is multicast.
//
// O is only rescaled when a row's running maximum grows by more than 2^8 (otherwise the stale
// reference maximum is kept; the final division by the row sum makes it exact).
// Query-side relocation: the first shared_kv_lens[b] keys are scored against queries rotated by
// the inverse shift, then each row block swaps its query tile for the plain one.
// Every mbarrier wait is bounded; on expiry the kernel raises the error flag, frees its TMEM
// and returns.
#include <type_traits>

#include "common.cuh"
#include "tcgen05.cuh"

namespace acache {

namespace tc {

namespace wide {

constexpr int BM = 128;       // rows per row block
constexpr int RB = 2;         // row blocks per CTA
constexpr int BN = 64;        // keys per tile
constexpr int NT_ROWS = RB * BM;             // row-owning threads (warps 0-7)
constexpr int W_ROWS = NT_ROWS / 32;
constexpr int W_ISSUE = W_ROWS;              // first issuing warp (one per row block)
constexpr int W_LOADK = W_ISSUE + RB;        // first K loader warp
constexpr int NT_LOAD = 64;                  // threads per loader group (K: warps 10,11; V: warps 12,13)
constexpr int W_LOADV = W_LOADK + NT_LOAD / 32;
constexpr int NT_ALL = (W_LOADV + NT_LOAD / 32) * 32;   // 448
constexpr int NSK = 3;        // K stages: K(i+1) is published, and S(i+1) issued, while the softmax of tile i runs
constexpr int NSV = 2;        // V stages
constexpr int RING = 8;       // tiles whose dead-key masks are kept for the row-owning warps
constexpr uint32_t kTmemCols = 512;
constexpr int kPairRows = 1024;   // virtual rows per request from which CTA pairs are used

template <typename T, typename TR, typename TC, int D, bool PAIR>
__global__ void __launch_bounds__(NT_ALL, 1) attention_tc256_kernel(
    const T* __restrict__ q, int64_t q_stride, T* __restrict__ out, int64_t o_stride, const T* __restrict__ k_cache,
    const T* __restrict__ v_cache, int64_t num_slots, int n_heads, int n_kv_heads, const int32_t* __restrict__ cu_q,
    const int32_t* __restrict__ cu_k, const int32_t* __restrict__ slot_map, const int32_t* __restrict__ block_tables,
    int table_stride, int block_size, float scale_log2, const int32_t* __restrict__ shared_kv_lens,
    const int32_t* __restrict__ affix_shifts, const TR* __restrict__ rope_cos, const TR* __restrict__ rope_sin,
    int64_t rope_stride, int rope_rows, int32_t* err_flag) {
  static_assert(!PAIR || D == 128, "a CTA of a pair stages one 64-column plane of V");
  constexpr int NC = PAIR ? 2 : 1;                // CTAs that work as one
  constexpr int CH = D * (int)sizeof(T) / 16;     // 16-byte chunks per row
  constexpr int KROWS = BN / NC;                  // keys of a tile whose K rows this CTA stages
  constexpr int VCH = CH / NC;                    // chunks of every V row this CTA stages
  constexpr int Q_BYTES = BM * D * (int)sizeof(T);      // one row block
  constexpr int K_BYTES = KROWS * D * (int)sizeof(T);
  constexpr int V_BYTES = BN * VCH * 16;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled operand layout needs 1024-byte aligned atoms
    if (threadIdx.x == 0 && err_flag) atomicExch(err_flag, 6);
    return;
  }
  uint8_t* sQ = smem;                    // RB blocks
  uint8_t* sK = sQ + RB * Q_BYTES;       // NSK stages
  uint8_t* sV = sK + NSK * K_BYTES;      // NSV stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + NSV * V_BYTES);
  // K landed [NSK], V landed [NSV], then S done [r][b] (4), P written [r][b] (4), P V done [r][tile parity] (4), Q in place [r] (2)
  constexpr int NBAR = NSK + NSV + 14;
  uint32_t* ring_words = reinterpret_cast<uint32_t*>(bars + ((NBAR + 1) & ~1));   // 16-byte aligned
  uint32_t* tmem_slot = ring_words + RING * 4;
  volatile int* give_up = reinterpret_cast<volatile int*>(tmem_slot + 1);   // set by the first role whose bounded wait runs out
  // per tile of the ring, 16 aligned bytes written and read with one instruction: which keys take no
  // part (two words) and the tile's number + 1
  const uint32_t dead_ring = smem_u32(ring_words);   // [RING tiles][4 words]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = n_heads / n_kv_heads;
  const int kv_row = n_kv_heads * D;
  const bool query_side = shared_kv_lens != nullptr && affix_shifts != nullptr;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;    // the first CTA of a pair issues its products

  // A pair's two CTAs are neighbours in x.  Without pairs the row tile is the slowest grid index,
  // so that the CTAs of every request's last, partly filled tile are handed out last and fill the
  // gaps of the final round instead of each delaying a full one behind it
  const int b = blockIdx.y, kvh = PAIR ? blockIdx.z : blockIdx.x;
  const int tile = PAIR ? blockIdx.x : blockIdx.z, m0 = tile * (RB * BM);
  const int m0_all = PAIR ? (tile & ~1) * (RB * BM) : m0;   // first row of the pair
  const int q0 = cu_q[b];
  const int vrows = (cu_q[b + 1] - q0) * g;
  if (m0_all >= vrows) return;
  const int kv0 = cu_k[b], kv_len = max(cu_k[b + 1] - kv0, 0);
  int shift = 0;
  if (query_side) {
    shift = affix_shifts[b];
    if (shift < 0 || shift >= rope_rows) {
      if (tid == 0 && err_flag) atomicExch(err_flag, 4);
      shift = 0;
    }
  }
  // shared_kv_lens splits the keys in two runs that are tiled separately; with affix_shifts the
  // first run is scored against inverse-rotated queries
  int n_shared = 0;
  if (shared_kv_lens != nullptr) n_shared = min(max(shared_kv_lens[b], 0), kv_len);
  const int nt0 = (n_shared + BN - 1) / BN;
  const int nt1 = (kv_len - n_shared + BN - 1) / BN;
  const int n_tiles = nt0 + nt1;
  // the queries are swapped for the plain ones before tile nt0 is scored
  const bool start_rotated = query_side && nt0 > 0;
  const bool swaps = start_rotated && nt1 > 0;

  const bool is_row = warp < W_ISSUE, is_issuer = warp >= W_ISSUE && warp < W_LOADK;
  // this thread's row (issuing warps: the row block they issue for)
  const int rb = is_row ? warp >> 2 : (is_issuer ? warp - W_ISSUE : 0);
  const int brow = tid & (BM - 1);                 // row inside the block = TMEM lane
  const int vr = m0 + tid;
  const bool row_ok = is_row && vr < vrows;
  const int qi = row_ok ? vr / g : 0;
  const int head = kvh * g + (row_ok ? vr % g : 0);
  T* out_row = out + ((int64_t)q0 + qi) * o_stride + (int64_t)head * D;

  if (n_tiles == 0) {  // no keys: zeros
    if (row_ok) {
      for (int c = 0; c < CH; ++c) *reinterpret_cast<uint4*>(out_row + c * (16 / sizeof(T))) = make_uint4(0, 0, 0, 0);
    }
    return;
  }

  const uint32_t bar_k = smem_u32(&bars[0]), bar_v = smem_u32(&bars[NSK]), bar_s = smem_u32(&bars[NSK + NSV]),
                 bar_p = smem_u32(&bars[NSK + NSV + 4]), bar_o = smem_u32(&bars[NSK + NSV + 8]),
                 bar_q = smem_u32(&bars[NSK + NSV + 12]);
  if (tid == 0) {
    // one arrival per warp; the barriers the issuing threads wait on take both CTAs' arrivals
    for (int s = 0; s < NSK; ++s) mbar_init(bar_k + s * 8, NC * NT_LOAD / 32);
    for (int s = 0; s < NSV; ++s) mbar_init(bar_v + s * 8, NC * NT_LOAD / 32);
    for (int s = 0; s < 4; ++s) {
      mbar_init(bar_s + s * 8, 1);
      mbar_init(bar_p + s * 8, NC * BM / 32);
      mbar_init(bar_o + s * 8, 1);
    }
    for (int r = 0; r < RB; ++r) mbar_init(bar_q + r * 8, NC * BM / 32);
    *give_up = 0;
    for (int t = 0; t < RING; ++t) ring_words[t * 4 + 2] = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();          // both CTAs' barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;   // the whole TMEM of the SM: column 0 in both CTAs of a pair
  const uint32_t t_lane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
  const uint32_t col_s = (uint32_t)rb * 256u, col_o = (uint32_t)rb * 256u + 128u;

  // bounded wait that also ends when another role has given up
  auto wait_bar = [&](uint32_t bar, uint32_t parity) -> bool {
    const long long t0 = clock64();
    for (uint32_t it = 0;; ++it) {
      uint32_t done;
      asm volatile(
          "{\n\t.reg .pred p;\n\t"
          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(done) : "r"(bar), "r"(parity) : "memory");
      if (done) return true;
      if ((it & 63) == 63) {
        if (*give_up) return false;
        if (clock64() - t0 > kWaitCycles) {
          *give_up = 1;
          return false;
        }
        __nanosleep(32);
      }
    }
  };
  auto arrive = [&](uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); };
  // arrival on the barrier at this offset in CTA `to` of the pair.  A cluster-scope release costs
  // about a thousand cycles here; the plain form is what the data needs: it lies in this CTA's own
  // shared memory and has been made visible to the tensor cores by the proxy fence before
  auto arrive_at = [&](uint32_t bar, uint32_t to) {
    if (PAIR && to != rank) asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(map_to_cta(bar, to)) : "memory");
    else arrive(bar);
  };
  // one arrival for the whole warp, on the barrier at this offset in the first CTA of the pair
  auto warp_arrive_first = [&](uint32_t bar) {
    __syncwarp();
    if (lane == 0) arrive_at(bar, 0);
  };
  // what this thread wrote to its CTA's shared memory becomes visible to the tensor cores
  auto publish_fence = [&]() { fence_proxy_async(); };
  // tile t's event on a pair of barriers that alternate with the tile's parity: barrier t & 1,
  // its (t >> 1)-th completion (S(t) done, P(t) written, P V(t) done)
  auto wait_tile = [&](uint32_t bar, int t) { return wait_bar(bar + (t & 1) * 8, (uint32_t)((t >> 1) & 1)); };
  // barrier of the row-owning threads only
  auto rows_sync = [&]() { asm volatile("bar.sync 1, %0;" ::"n"(NT_ROWS) : "memory"); };

  // a warp is live when at least one of its 32 rows is a real (query, head) pair
  const bool warp_live = is_row && m0 + warp * 32 < vrows;
  // a row block of the products is live when it has a real row in any of the CTAs that share it
  const bool block_live = m0_all + rb * BM < vrows;

  if (is_issuer) {
    // ---- the issuing thread of row block rb (first CTA of a pair only) --------------------------
    if (lane == 0 && rank == 0) {
      const uint32_t idesc_s = make_idesc(Fmt<T>::id, 0, BN, NC * BM);
      const uint32_t idesc_o = make_idesc(Fmt<T>::id, 1, D, NC * BM);
      const uint32_t qb = smem_u32(sQ) + rb * Q_BYTES;
      const uint32_t my_s = bar_s + rb * 16, my_p = bar_p + rb * 16, my_o = bar_o + rb * 16, my_q = bar_q + rb * 8;
      auto product = [&](uint32_t d, uint64_t ad, uint64_t bd, uint32_t idesc, uint32_t acc) {
        if (PAIR) mma_ss_pair(d, ad, bd, idesc, acc);
        else mma_ss(d, ad, bd, idesc, acc);
      };
      auto done_on = [&](uint32_t bar) {   // arrives on the barrier (of every CTA) when the products so far are done
        if (!block_live) {                 // a row block of padding only: no product, the hand-over stays
          arrive(bar);
          if (PAIR) arrive_at(bar, 1);
        } else if (PAIR) {
          mma_commit_pair(bar);
        } else {
          mma_commit(bar);
        }
      };
      auto issue_s = [&](int i) {   // S(i) = Q K(i)^T into S buffer i & 1
        if (block_live) {
          const uint32_t kb = smem_u32(sK) + (i % NSK) * K_BYTES;
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t a_off = (ks / 4) * (BM * 128) + (ks % 4) * 32;
            const uint32_t b_off = (ks / 4) * (KROWS * 128) + (ks % 4) * 32;
            product(tmem_base + col_s + (i & 1) * BN, make_desc(qb + a_off, 16, 1024), make_desc(kb + b_off, 16, 1024),
                    idesc_s, ks > 0 ? 1u : 0u);
          }
        }
        done_on(my_s + (i & 1) * 8);
      };
      bool ok = wait_bar(my_q, 0);
      ok = wait_bar(bar_k, 0) && ok;
      tc_fence_after();
      if (ok) issue_s(0);
      for (int i = 0; i < n_tiles && ok; ++i) {
        if (i + 1 < n_tiles) {
          // S buffer (i+1)&1 held S(i-1), read before P(i-1) was published, which was awaited
          if (swaps && i + 1 == nt0) ok = wait_bar(my_q, 1);   // the plain queries are in place
          ok = wait_bar(bar_k + ((i + 1) % NSK) * 8, (uint32_t)(((i + 1) / NSK) & 1)) && ok;
          tc_fence_after();
          if (!ok) break;
          issue_s(i + 1);
        }
        ok = wait_tile(my_p, i);
        ok = wait_bar(bar_v + (i % NSV) * 8, (uint32_t)((i / NSV) & 1)) && ok;
        tc_fence_after();
        if (!ok) break;
        if (block_live) {
          const uint32_t vb = smem_u32(sV) + (i % NSV) * V_BYTES;
#pragma unroll
          for (int ks = 0; ks < BN / 16; ++ks) {
            // A = P(i): 16 keys = 8 columns of S buffer i & 1, which the softmax overwrote with its weights
            const uint32_t pa = tmem_base + col_s + (i & 1) * BN + ks * 8;
            if (PAIR) mma_ts_pair(tmem_base + col_o, pa, make_desc(vb + ks * 2048, BN * 128, 1024), idesc_o, (i > 0 || ks > 0) ? 1u : 0u);
            else mma_ts(tmem_base + col_o, pa, make_desc(vb + ks * 2048, BN * 128, 1024), idesc_o, (i > 0 || ks > 0) ? 1u : 0u);
          }
        }
        done_on(my_o + (i & 1) * 8);
      }
    }
  } else if (!is_row) {
    // ---- loader warps: one group gathers this CTA's part of the K tiles, the other of the V tiles -
    const bool for_k = warp < W_LOADV;
    const int ltid = tid - (for_k ? W_LOADK : W_LOADV) * 32;     // 0 .. NT_LOAD - 1
    // K: KROWS keys x CH chunks; V: BN keys x VCH chunks
    constexpr int K_ITER = KROWS * CH / NT_LOAD, K_RPI = NT_LOAD / CH;
    constexpr int V_ITER = BN * VCH / NT_LOAD, V_RPI = NT_LOAD / VCH;
    static_assert(K_RPI <= 32 && 32 % K_RPI == 0 && V_RPI <= 32 && 32 % V_RPI == 0, "the rows of one iteration lie in one half of the tile");
    // keys [j0, j_end) of the tile's run
    auto tile_span = [&](int i, int& j0, int& j_end) {
      if (i < nt0) {
        j0 = i * BN;
        j_end = n_shared;
      } else {
        j0 = n_shared + (i - nt0) * BN;
        j_end = kv_len;
      }
    };
    // Entry codes: >= 0 a slot, -1 a key that takes no part, -2 an entry outside the cache
    // (reported), -3 past the end of the run.  Lane l holds rows l and l + 32 of the tile.  The
    // words are only LOADED by fetch_raw, tiles ahead, and looked at when the tile is gathered.
    auto fetch_raw = [&](int i, int32_t (&raw)[2]) {
      int j0, j_end;
      tile_span(i, j0, j_end);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int j = j0 + h * 32 + lane;
        int32_t v = 0;
        if (j < j_end) v = slot_map ? slot_map[kv0 + j] : block_tables[(int64_t)b * table_stride + j / block_size];
        raw[h] = v;
      }
    };
    auto interpret = [&](int i, const int32_t (&raw)[2], int32_t& e0, int32_t& e1) {
      int j0, j_end;
      tile_span(i, j0, j_end);
      int32_t code[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int j = j0 + h * 32 + lane;
        code[h] = -3;
        if (j < j_end) {
          int64_t slot = raw[h];
          if (slot_map) {
            code[h] = slot == -1 ? -1 : ((slot < 0 || slot >= num_slots) ? -2 : (int32_t)slot);
          } else {
            slot = slot < 0 ? -2 : slot * block_size + j % block_size;
            code[h] = (slot < 0 || slot >= num_slots) ? -2 : (int32_t)slot;  // fits 32 bits: the dispatcher refuses larger caches
          }
        }
      }
      e0 = code[0];
      e1 = code[1];
      if (for_k) {   // the K group also publishes the tile's dead keys and reports bad entries
        const uint32_t dead_lo = __ballot_sync(0xFFFFFFFFu, code[0] < 0), dead_hi = __ballot_sync(0xFFFFFFFFu, code[1] < 0);
        if (warp == W_LOADK && lane == 0) {   // the slot held tile i - RING, whose softmax ended several products ago
          asm volatile("st.volatile.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dead_ring + (i % RING) * 16), "r"(dead_lo),
                       "r"(dead_hi), "r"((uint32_t)i + 1u), "r"(0u) : "memory");
        }
        if (err_flag && (code[0] == -2 || code[1] == -2)) atomicExch(err_flag, 3);
      }
    };
    auto load_k = [&](int i, int32_t e0, int32_t e1) {
      const uint32_t base = smem_u32(sK) + (i % NSK) * K_BYTES;
      const int my_c = ltid % CH, my_r = ltid / CH;
#pragma unroll
      for (int it = 0; it < K_ITER; ++it) {
        const int r = my_r + it * K_RPI;                  // row of this CTA's part = key rank * KROWS + r of the tile
        const int key = PAIR ? (int)rank * KROWS + r : r;
        int64_t slot = __shfl_sync(0xFFFFFFFFu, PAIR ? (rank == 0 ? e0 : e1) : ((it * K_RPI < 32) ? e0 : e1), key & 31);
        const bool ok = slot >= 0;
        if (!ok) slot = 0;
        cp_async16(base + swz<D>(KROWS, r, my_c), k_cache + slot * kv_row + (int64_t)kvh * D + my_c * (16 / sizeof(T)), ok);
      }
    };
    auto load_v = [&](int i, int32_t e0, int32_t e1) {
      const uint32_t base = smem_u32(sV) + (i % NSV) * V_BYTES;
      const int my_c = ltid % VCH, my_r = ltid / VCH;
#pragma unroll
      for (int it = 0; it < V_ITER; ++it) {
        const int r = my_r + it * V_RPI;
        int64_t slot = __shfl_sync(0xFFFFFFFFu, (it * V_RPI < 32) ? e0 : e1, r & 31);
        const bool ok = slot >= 0;
        if (!ok) slot = 0;
        // this CTA's columns of the row: chunks rank * VCH .. + VCH - 1 (all of them without a pair)
        cp_async16(base + swz<D>(BN, r, my_c),
                   v_cache + slot * kv_row + (int64_t)kvh * D + ((int)rank * VCH + my_c) * (16 / sizeof(T)), ok);
      }
    };
    const uint32_t bar_land = for_k ? bar_k : bar_v;
    const uint32_t bar_read = for_k ? bar_s : bar_o;   // the products that read a stage, per row block
    const int nst = for_k ? NSK : NSV;
    int32_t raw_now[2], raw_a[2] = {0, 0}, raw_b[2] = {0, 0};   // lookups of tiles i, i + 1 and i + 2 in flight
    fetch_raw(0, raw_now);
    if (1 < n_tiles) fetch_raw(1, raw_a);
    if (2 < n_tiles) fetch_raw(2, raw_b);
    bool ok = true;
    for (int i = 0; i < n_tiles; ++i) {
      // the stage of tile i held tile i - nst, whose last readers are products of both row blocks
      if (i >= nst) {
        ok = wait_tile(bar_read, i - nst) && ok;
        ok = wait_tile(bar_read + 16, i - nst) && ok;
        if (!ok) break;
      }
      int32_t e0, e1;
      interpret(i, raw_now, e0, e1);
      if (for_k) load_k(i, e0, e1);
      else load_v(i, e0, e1);
      cp_async_commit();
      raw_now[0] = raw_a[0];
      raw_now[1] = raw_a[1];
      raw_a[0] = raw_b[0];
      raw_a[1] = raw_b[1];
      if (i + 3 < n_tiles) fetch_raw(i + 3, raw_b);
      if (i > 0) {
        cp_async_wait<1>();                    // tile i - 1 has landed for this thread
        publish_fence();
        warp_arrive_first(bar_land + ((i - 1) % nst) * 8);
      }
    }
    cp_async_wait<0>();
    publish_fence();
    if (ok) warp_arrive_first(bar_land + ((n_tiles - 1) % nst) * 8);
    else *give_up = 1;
  } else {
    // ---- the threads that own the rows ----------------------------------------------------------
    const uint32_t my_s = bar_s + rb * 16, my_p = bar_p + rb * 16, my_o = bar_o + rb * 16, my_q = bar_q + rb * 8;
    // the 128 threads of a row block load its query tile
    auto load_q = [&](bool rotated) {
      uint8_t* dstb = sQ + rb * Q_BYTES;
      for (int id = brow; id < BM * CH; id += BM) {
        const int r = id / CH, c = id % CH;
        const int v = m0 + rb * BM + r;
        const bool ok = v < vrows;
        const int rq = ok ? v / g : 0, rh = kvh * g + (ok ? v % g : 0);
        const T* src = q + (int64_t)(q0 + rq) * q_stride + (int64_t)rh * D + c * (16 / sizeof(T));
        if (!rotated) {
          cp_async16(smem_u32(dstb) + swz<D>(BM, r, c), src, ok);
        } else if (c < CH / 2) {
          // q*cos - rotate_half(q)*sin for the chunk pair (d, d + D/2), rounded to T
          constexpr int E = 16 / sizeof(T);
          Vec16<T> a, bb, o1, o2;
          a.u = make_uint4(0, 0, 0, 0);
          bb.u = a.u;
          if (ok) {
            a.u = *reinterpret_cast<const uint4*>(src);
            bb.u = *reinterpret_cast<const uint4*>(src + D / 2);
          }
          const TR* cr = rope_cos + (int64_t)shift * rope_stride;
          const TR* sr = rope_sin + (int64_t)shift * rope_stride;
          const int d = c * E;
#pragma unroll
          for (int e = 0; e < E; ++e) {
            const float x1 = to_f32<T>(a.e[e]), x2 = to_f32<T>(bb.e[e]);
            o1.e[e] = from_f32<T>(rot_lo<TC>(x1, x2, to_f32<TR>(cr[d + e]), -to_f32<TR>(sr[d + e])));
            o2.e[e] = from_f32<T>(rot_hi<TC>(x1, x2, to_f32<TR>(cr[d + D / 2 + e]), -to_f32<TR>(sr[d + D / 2 + e])));
          }
          *reinterpret_cast<uint4*>(dstb + swz<D>(BM, r, c)) = o1.u;
          *reinterpret_cast<uint4*>(dstb + swz<D>(BM, r, c + CH / 2)) = o2.u;
        }
      }
    };
    load_q(start_rotated);
    cp_async_commit();
    cp_async_wait<0>();
    publish_fence();
    warp_arrive_first(my_q);

    float m_ref = -INFINITY, l_sum = 0.f;
    uint32_t s[BN];
    bool ok = true;
    for (int i = 0; i < n_tiles; ++i) {
      ok = wait_tile(my_s, i) && ok;
      tc_fence_after();
      // query tile swap at the partition boundary: S(i) was the last product against the rotated
      // queries; the issuing thread holds S(i+1) back until the plain ones are in place
      if (swaps && i + 1 == nt0) {
        load_q(false);
        cp_async_commit();
        cp_async_wait<0>();
        publish_fence();
        warp_arrive_first(my_q);
      }
      if (warp_live) {
        // ---- scores of this thread's row and their maximum ----
        tmem_ld32(t_lane + col_s + (i & 1) * BN, s);
        tmem_ld32(t_lane + col_s + (i & 1) * BN + 32, s + 32);
        // while the scores are on their way: the tile's dead keys, published by this CTA's K loader
        // long before the product that was awaited, and P buffer i & 1, free once P V(i-2) is done
        uint32_t dl, dh, tag, pad;
        auto read_ring = [&]() {
          asm volatile("ld.volatile.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(dl), "=r"(dh), "=r"(tag), "=r"(pad)
                       : "r"(dead_ring + (i % RING) * 16) : "memory");
        };
        read_ring();
        if (tag != (uint32_t)i + 1u) {
          const long long t0 = clock64();
          while (tag != (uint32_t)i + 1u && clock64() - t0 < kWaitCycles && !*give_up) {
            __nanosleep(32);
            read_ring();
          }
          if (tag != (uint32_t)i + 1u) ok = false;
        }
        float mx = -INFINITY;
        tmem_wait_ld();
        if ((dl | dh) != 0u) {   // a tile with keys that take no part (holes, the end of a run)
          const uint64_t dead = (((uint64_t)dh) << 32) | dl;
#pragma unroll
          for (int c = 0; c < BN; ++c) {
            const float v = ((dead >> c) & 1ull) ? -INFINITY : __uint_as_float(s[c]);
            s[c] = __float_as_uint(v);
            mx = fmaxf(mx, v);
          }
        } else {
          float m8[8];   // eight independent chains of three-input maxima
#pragma unroll
          for (int k = 0; k < 8; ++k) m8[k] = fmaxf(__uint_as_float(s[2 * k]), __uint_as_float(s[2 * k + 1]));
#pragma unroll
          for (int c = 16; c < BN; c += 16) {
#pragma unroll
            for (int k = 0; k < 8; ++k) m8[k] = max3(m8[k], __uint_as_float(s[c + 2 * k]), __uint_as_float(s[c + 2 * k + 1]));
          }
          mx = max3(max3(m8[0], m8[1], m8[2]), max3(m8[3], m8[4], m8[5]), fmaxf(m8[6], m8[7]));
        }
        mx *= scale_log2;
        const bool grow = mx > m_ref + 8.0f;  // also true on the first tile with a live key (m_ref = -inf)
        // ---- lazy rescale of O, weights, P ----
        if (__any_sync(0xFFFFFFFFu, grow) && i > 0) {
          // O may only be touched between two products: P V(i-1) done, and P V(i) is not issued
          // before this thread publishes P(i)
          ok = wait_tile(my_o, i - 1) && ok;
          tc_fence_after();
          const float f = grow ? ex2(m_ref - mx) : 1.0f;
          l_sum *= f;
          uint32_t o[32];
#pragma unroll 1
          for (int c0 = 0; c0 < D; c0 += 32) {
            tmem_ld32(t_lane + col_o + c0, o);
            tmem_wait_ld();
#pragma unroll
            for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * f);
            tmem_st32(t_lane + col_o + c0, o);
          }
          tmem_wait_st();
        }
        if (grow) m_ref = mx;
        const float m_use = m_ref == -INFINITY ? 0.f : m_ref;   // no live key so far: every p is 0
        // two scores per packed fma, two partial row sums per packed add
        const uint64_t sc2 = pack_f32x2(scale_log2, scale_log2), nm2 = pack_f32x2(-m_use, -m_use);
        uint64_t rs2 = pack_f32x2(0.f, 0.f);
        uint32_t w[BN / 2];   // the row's weights, two per word
#pragma unroll
        for (int c = 0; c < BN; c += 2) {
          float x0, x1;
          unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(s[c]), __uint_as_float(s[c + 1])), sc2, nm2), x0, x1);
          const float p0 = ex2(x0), p1 = ex2(x1);
          rs2 = add_f32x2(rs2, pack_f32x2(p0, p1));
          w[c / 2] = pack2<T>(p0, p1);
        }
        // P(i) takes the place of the first 32 columns of S(i) in TMEM, where the P V product reads it
        tmem_st32(t_lane + col_s + (i & 1) * BN, w);
        tmem_wait_st();
        float r0, r1;
        unpack_f32x2(rs2, r0, r1);
        l_sum += r0 + r1;
      }
      tc_fence_before();
      warp_arrive_first(my_p + (i & 1) * 8);
      if (!ok) break;
    }
    if (ok) ok = wait_tile(my_o, n_tiles - 1);
    tc_fence_after();
    if (!ok) *give_up = 1;
    rows_sync();
    const bool failed = *give_up != 0;

    if (failed) {
      if (tid == 0 && err_flag) atomicExch(err_flag, 5);
    } else if (warp_live) {
      // thread = row: divide by the row sum and write
      const float inv = l_sum > 0.f ? 1.0f / l_sum : 0.f;
      uint32_t o[32];
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        tmem_ld32(t_lane + col_o + c0, o);
        tmem_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            uint4 w;
            w.x = pack2<T>(__uint_as_float(o[c]) * inv, __uint_as_float(o[c + 1]) * inv);
            w.y = pack2<T>(__uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv);
            w.z = pack2<T>(__uint_as_float(o[c + 4]) * inv, __uint_as_float(o[c + 5]) * inv);
            w.w = pack2<T>(__uint_as_float(o[c + 6]) * inv, __uint_as_float(o[c + 7]) * inv);
            *reinterpret_cast<uint4*>(out_row + c0 + c) = w;
          }
        }
      }
    }
  }
  cp_async_wait<0>();
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();          // the other CTA no longer reads this CTA's shared memory or barriers
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

template <typename T, typename TR> struct PromoteT { using type = float; };
template <> struct PromoteT<__half, __half> { using type = __half; };
template <> struct PromoteT<__nv_bfloat16, __nv_bfloat16> { using type = __nv_bfloat16; };

template <typename T, typename TR, int D, bool PAIR>
static int launch(const AttnArgs& a) {
  using TC = typename PromoteT<T, TR>::type;
  constexpr int NC = PAIR ? 2 : 1;
  constexpr size_t smem = RB * BM * D * sizeof(T) + (NSK + NSV) * (BN / NC) * D * sizeof(T) + 512;
  const int g = a.n_heads / a.n_kv_heads;
  const bool relocate = a.shared_prefix_len > 0 && a.affix_shifts != nullptr;
  const int rows_per_launch_unit = NC * RB * BM;
  const int tiles = NC * ((a.max_q * g + rows_per_launch_unit - 1) / rows_per_launch_unit);
  const dim3 grid = PAIR ? dim3(tiles, a.batch, a.n_kv_heads) : dim3(a.n_kv_heads, a.batch, tiles);
  auto kern = attention_tc256_kernel<T, TR, TC, D, PAIR>;
  ACACHE_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  cudaLaunchConfig_t lc = {};
  lc.gridDim = grid;
  lc.blockDim = dim3(NT_ALL);
  lc.dynamicSmemBytes = smem;
  lc.stream = a.st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = NC;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  lc.attrs = at;
  lc.numAttrs = PAIR ? 1 : 0;
  ACACHE_CUDA_CHECK(cudaLaunchKernelEx(
      &lc, kern, (const T*)a.q, a.q_stride, (T*)a.out, a.o_stride, (const T*)a.k_cache, (const T*)a.v_cache, a.num_slots,
      a.n_heads, a.n_kv_heads, a.cu_q, a.cu_k, a.slot_map, a.block_tables, a.table_stride, a.block_size,
      a.scale * 1.4426950408889634f, a.shared_kv_lens, relocate ? a.affix_shifts : (const int32_t*)nullptr,
      (const TR*)a.rope_cos, (const TR*)a.rope_sin, a.rope_stride, a.rope_rows, a.err_flag));
  ACACHE_LAUNCH_CHECK();
  return ACACHE_OK;
}

template <typename T, typename TR>
static int by_dim(const AttnArgs& a) {
  const int g = a.n_heads / a.n_kv_heads;
  if (a.head_dim == 128) {
    // a pair of CTAs per 512 rows: a few per cent faster when the rows fill the pairs (measured at
    // 3400 and 8192 rows), slower when a request's last pair is mostly padding
    if (a.max_q * g >= kPairRows) return launch<T, TR, 128, true>(a);
    return launch<T, TR, 128, false>(a);
  }
  if (a.head_dim == 64) return launch<T, TR, 64, false>(a);
  return ACACHE_EUNSUPPORTED;
}

}  // namespace wide

}  // namespace tc

// The 256-row kernel takes requests with more than 128 virtual rows whose keys are not relocated
// while they are staged; the caller has checked dtypes, head size, alignment and cache size.
int attention_tc256_dispatch(const AttnArgs& a, int dtype, int rope_dtype) {
  using namespace tc::wide;
  const int g = a.n_heads / a.n_kv_heads;
  const bool relocate = a.shared_prefix_len > 0 && a.affix_shifts != nullptr;
  if (relocate && a.shared_kv_lens == nullptr) return ACACHE_EUNSUPPORTED;   // key-side relocation
  if (a.max_q * g <= BM) return ACACHE_EUNSUPPORTED;
  if (dtype == ACACHE_BF16) {
    if (rope_dtype == ACACHE_F32) return by_dim<__nv_bfloat16, float>(a);
    if (rope_dtype == ACACHE_BF16) return by_dim<__nv_bfloat16, __nv_bfloat16>(a);
    return by_dim<__nv_bfloat16, __half>(a);
  }
  if (rope_dtype == ACACHE_F32) return by_dim<__half, float>(a);
  if (rope_dtype == ACACHE_F16) return by_dim<__half, __half>(a);
  return by_dim<__half, __nv_bfloat16>(a);
}

}  // namespace acache

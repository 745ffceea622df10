// Bidirectional varlen attention over the slot-mapped paged cache on the 5th-generation
// tensor cores (tcgen05) with TMEM accumulators, for bf16/fp16 and head_dim 64/128.
//
// One CTA = one (request, KV head, tile of 128 "virtual rows").  A virtual row is a
// (query, head-of-the-GQA-group) pair, so all query heads that share a KV head share one
// pass over its K/V.  Roles inside the CTA, handing over through mbarriers only:
//   warps 0-3  own the rows: thread t owns row t (TMEM lane t): tcgen05.ld of its scores,
//              online softmax in the exp2 domain, the weights P written back to TMEM over the
//              scores (two per 32-bit column), where the P V product reads its A operand;
//              they also stage K/V, unless (block decode) warps 5-8 do that for them;
//   warp 4     one thread issues every tcgen05.mma: S(i+1) = Q K(i+1)^T as soon as K(i+1)
//              has landed, one tile ahead of the softmax, into one of two S buffers in TMEM,
//              and O += P(i) V(i) as soon as P(i) is written;
//   warps 5-8  (LOADERS, requests of at most 32 virtual rows) stage K/V and publish which
//              rows of a tile take no part.
// Per tile of 64 keys:
//   * the tile's 64 slot-map entries (two per lane) are loaded three tiles ahead and looked
//     at one iteration later, so nothing waits for a lookup; an entry of -1 is a key that
//     takes no part (its row is zero-filled and its score masked);
//   * K and V rows are gathered with 16-byte cp.async into shared memory in the
//     128-byte-swizzled layout the MMA descriptors expect (Q/K/P K-major, V MN-major), two
//     stages each; a stage is refilled as soon as its last reader (the S product for K, the
//     P V product for V) is done;
//   * S and O are fp32 in TMEM (256 columns per CTA, two CTAs per SM).
// Requests of at most 32 virtual rows (COPIES = 4): the rows are staged four times and warp w
// runs the softmax of key columns 16w..16w+15 only; the four slices are folded at the end.
// O is only rescaled when a row's running maximum grows by more than 2^8 (otherwise the
// stale reference maximum is kept; the final division by the row sum makes it exact).
// Query-side relocation: the first shared_kv_lens[b] keys are scored against queries
// rotated by the inverse shift, then the query tile is swapped for the plain one.
// Key-side relocation: keys of the shared span are rotated while they are staged.
//
// Shared-span grouping (SPLIT = true, block decode): when every request has at most 32
// virtual rows and the first shared_kv_lens[b] entries of all requests name the same slots
// (up to holes), one CTA = (two consecutive requests, KV head): warps 2r and 2r + 1 hold two
// copies of the 32 rows of request r and split a tile's key columns between them, as the
// per-request kernel does with four copies.  The CTA first walks the shared span, staged ONCE
// for both requests (slot = the union of their entries, each warp masks its own request's
// holes), then the remaining keys of request 0, then of request 1: a tile of one request is
// dead for the other's warps (their P rows are zero).  The products of a 64-key tile cost the
// same however many of their 128 rows are distinct, so the span costs half the tensor-core
// instructions and half the L2 -> shared-memory traffic, and a launch has half the CTAs, each
// paying its set-up once; two CTAs still share an SM and hide each other's waits.  (The code
// also instantiates as four requests with one copy each, COPIES = 1; one CTA per SM was slower.)
// Every mbarrier wait is bounded; on expiry the kernel raises the error flag, frees its
// TMEM and returns.
#include <type_traits>

#include "common.cuh"
#include "tcgen05.cuh"

namespace acache {

// implemented in attention_tc256.cu: requests of more than 128 virtual rows, 256 rows per CTA
int attention_tc256_dispatch(const AttnArgs& a, int dtype, int rope_dtype);

namespace tc {

constexpr int BM = 128;      // virtual rows per CTA
constexpr int BN = 64;       // keys per tile
constexpr int NT = 128;      // threads that stage K/V and own the rows (warps 0-3)
constexpr int NT_ALL = 160;  // + warp 4, whose first lane issues every tensor-core product
constexpr int NT_LOAD = 288; // + warps 5-8 that take the K/V staging over from the row-owning warps (LOADERS)
constexpr int GROUP = 4;     // row-owning warps = most requests a work item can hold
constexpr int kGroupedRequests = 2;   // requests per work item of the grouped kernel as launched (two warps each)
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColS = 0, kColO = 128;

struct SplitArgs {
  int n_items_a;        // work items = ceil(batch / requests per item) * n_kv_heads
  int batch;
};

template <typename T, typename TR, typename TC, int D, bool KEYSIDE, bool SPLIT, int COPIES, bool LOADERS>
__global__ void __launch_bounds__(LOADERS ? NT_LOAD : NT_ALL, 2) attention_tc_kernel(
    const T* __restrict__ q, int64_t q_stride, T* __restrict__ out, int64_t o_stride, const T* __restrict__ k_cache,
    const T* __restrict__ v_cache, int64_t num_slots, int n_heads, int n_kv_heads, const int32_t* __restrict__ cu_q,
    const int32_t* __restrict__ cu_k, const int32_t* __restrict__ slot_map, const int32_t* __restrict__ block_tables,
    int table_stride, int block_size, float scale_log2, int shared_prefix_len,
    const int32_t* __restrict__ shared_kv_lens,
    const int32_t* __restrict__ affix_shifts, const TR* __restrict__ rope_cos, const TR* __restrict__ rope_sin,
    int64_t rope_stride, int rope_rows, int32_t* err_flag, SplitArgs sp) {
  constexpr int CH = D * (int)sizeof(T) / 16;     // 16-byte chunks per row
  // requests per work item, and copies of a request's (at most 32) rows among the 128 rows of the
  // products: every copy runs the softmax of 1 / CP of a tile's key columns.  Plain kernel: one
  // request, COPIES copies; grouped kernel: COPIES = 1 -> four requests, one copy each,
  // COPIES = 2 -> two requests, two copies each
  constexpr int GR = SPLIT ? (COPIES == 2 ? 2 : GROUP) : 1;
  constexpr int CP = SPLIT ? GROUP / GR : COPIES;
  constexpr int Q_BYTES = BM * D * (int)sizeof(T);
  constexpr int KV_BYTES = BN * D * (int)sizeof(T);

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  chain_release();
  chain_wait();
  if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled operand layout needs 1024-byte aligned atoms
    if (threadIdx.x == 0 && err_flag) atomicExch(err_flag, 6);
    return;
  }
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Q_BYTES;            // 2 stages
  uint8_t* sV = sK + 2 * KV_BYTES;       // 2 stages
  // mbarriers: [0],[1] K stage landed (128 arrivals); [2],[3] S buffer computed (tcgen05.commit);
  // [4],[5] P V(i) done (tcgen05.commit), barrier i & 1; [6],[7] V stage landed (128 arrivals, loader warps only);
  // [8],[9] P(i) written (and, without loader warps, V(i) landed) (128 arrivals), barrier i & 1: a
  // warp may publish P(i+1) before the others have published P(i), but not P(i+2), whose scores
  // are only issued once P(i) is complete
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + 2 * KV_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  // per request of the item (one unless this is a kind-A item): first query row, virtual
  // rows, first slot-map entry, rotation row
  int* rq_q0 = reinterpret_cast<int*>(tmem_slot + 1);
  int* rq_vrows = rq_q0 + GROUP;
  int* rq_kv0 = rq_vrows + GROUP;
  int* rq_shift = rq_kv0 + GROUP;
  volatile int* give_up = rq_shift + GROUP;   // set by the first role whose bounded wait runs out
  // rows of a tile that take no part, published by the loader warps for the row-owning warps
  volatile uint32_t* dead_ring = reinterpret_cast<volatile uint32_t*>(give_up + 1);   // [4 tiles][4 warps][2]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool is_loader = LOADERS && warp >= 5;
  const int ltid = is_loader ? tid - NT_ALL : tid;   // index among the 128 threads that stage K/V
  const int g = n_heads / n_kv_heads;
  const int kv_row = n_kv_heads * D;
  const bool query_side = shared_kv_lens != nullptr && affix_shifts != nullptr;

  // ---- which work item ----------------------------------------------------------------------
  int b, kvh, m0;
  const bool kind_a = SPLIT;       // an item of several requests
  if (SPLIT) {
    m0 = 0;
    b = ((int)blockIdx.x / n_kv_heads) * GR;
    kvh = (int)blockIdx.x % n_kv_heads;
  } else {
    b = blockIdx.y;
    kvh = blockIdx.z;
    m0 = blockIdx.x * BM;
  }
  const int n_req = kind_a ? min(GR, sp.batch - b) : 1;
  if (tid < GROUP) {
    int q0r = 0, vr = 0, kv0r = 0, sh = 0;
    if (tid < n_req) {
      q0r = cu_q[b + tid];
      vr = (cu_q[b + tid + 1] - q0r) * g;
      kv0r = cu_k[b + tid];
      if (query_side) {
        sh = affix_shifts[b + tid];
        if (sh < 0 || sh >= rope_rows) {
          if (err_flag) atomicExch(err_flag, 4);
          sh = 0;
        }
      }
    }
    rq_q0[tid] = q0r;
    rq_vrows[tid] = vr;
    rq_kv0[tid] = kv0r;
    rq_shift[tid] = sh;
  }
  const int kv0 = cu_k[b], kv_len = max(cu_k[b + 1] - kv0, 0);
  // shared_kv_lens splits the keys in two runs that are tiled separately; with affix_shifts the
  // first run is scored against inverse-rotated queries (query-side relocation)
  int n_shared = 0;
  if (shared_kv_lens != nullptr) n_shared = min(max(shared_kv_lens[b], 0), kv_len);
  if (kind_a) {
    for (int r = 1; r < n_req; ++r)  // grouping contract: one span length for the whole group
      if (min(max(shared_kv_lens[b + r], 0), max(cu_k[b + r + 1] - cu_k[b + r], 0)) != n_shared) {
        if (tid == 0 && err_flag) atomicExch(err_flag, 7);
      }
  }
  // tiles of the first run, then tiles of the second run (of a group: of its first request's
  // second run, then its second request's, ...; t0r[r] = first tile of request r's second run)
  const int nt0 = (n_shared + BN - 1) / BN;
  int t0r[GROUP + 1], klen[GROUP];
  t0r[0] = nt0;
#pragma unroll
  for (int r = 0; r < GROUP; ++r) {
    int kl = 0;
    if (r == 0) kl = kv_len;
    else if (SPLIT && r < n_req) kl = max(cu_k[b + r + 1] - cu_k[b + r], 0);
    klen[r] = kl;
    t0r[r + 1] = t0r[r] + ((r == 0 || SPLIT) ? (max(kl - n_shared, 0) + BN - 1) / BN : 0);
  }
  const int nt1 = t0r[GROUP] - nt0;
  const int n_tiles = nt0 + nt1;

  // COPIES = 4 (requests of at most 32 virtual rows, block decode): the 32 rows are staged four
  // times, copy w in rows 32w..32w+31, and warp w runs the softmax of key columns 16w..16w+15 of
  // every tile only (its P row is zero elsewhere), so each copy accumulates the attention over a
  // quarter of the keys with its own reference maximum; the four slices are folded at the end.
  // The tensor cores compute 128 rows either way; this spreads the softmax, the part that
  // bounds block decode, over all four warps.  A grouped item holds GR requests with CP = 4 / GR
  // copies each.
  const bool spread = CP > 1;
  // this thread's row: request slot ri of the item (copy ci of its rows), virtual row vr
  const int ri = kind_a ? (warp & 3) / CP : 0;
  const int ci = (warp & 3) % CP;
  const int vr = (kind_a || spread) ? lane : m0 + tid;

  const uint32_t bar_k = smem_u32(&bars[0]), bar_s = smem_u32(&bars[2]), bar_o = smem_u32(&bars[4]),
                 bar_v = smem_u32(&bars[6]), bar_p = smem_u32(&bars[8]);
  if (tid == 0) {
    mbar_init(bar_k, NT);
    mbar_init(bar_k + 8, NT);
    mbar_init(bar_s, 1);
    mbar_init(bar_s + 8, 1);
    mbar_init(bar_p, NT);
    mbar_init(bar_p + 8, NT);
    mbar_init(bar_o, 1);
    mbar_init(bar_o + 8, 1);
    mbar_init(bar_v, NT);
    mbar_init(bar_v + 8, NT);
    *give_up = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int my_vrows = rq_vrows[ri];
  int item_rows = 0;  // rows of the item that exist at all
#pragma unroll
  for (int r = 0; r < GROUP; ++r) item_rows = max(item_rows, rq_vrows[r]);
  if (!kind_a && m0 >= my_vrows) return;
  if (kind_a && item_rows == 0) return;
  const bool row_ok = vr < my_vrows;
  const int qi = row_ok ? vr / g : 0;
  const int head = kvh * g + (row_ok ? vr % g : 0);
  const int64_t q_row = (int64_t)rq_q0[ri] + qi;
  T* out_row = out + q_row * o_stride + (int64_t)head * D;

  if (n_tiles == 0) {  // no keys: zeros
    if (row_ok && tid < NT) {
      for (int c = 0; c < CH; ++c) *reinterpret_cast<uint4*>(out_row + c * (16 / sizeof(T))) = make_uint4(0, 0, 0, 0);
    }
    return;
  }

  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_lane = tmem_base + ((uint32_t)(warp * 32) << 16);

  // ---- loaders -----------------------------------------------------------------------
  auto load_q = [&](bool rotated) {
    // chunk id = it*NT + tid: 16 consecutive threads cover one row
    for (int id = ltid; id < BM * CH; id += NT) {
      const int r = id / CH, c = id % CH;
      const int rr = kind_a ? (r >> 5) / CP : 0;        // request slot of the row
      const int v = (kind_a || spread) ? (r & 31) : m0 + r;
      const bool ok = v < rq_vrows[rr];
      const int rq = ok ? v / g : 0, rh = kvh * g + (ok ? v % g : 0);
      const T* src = q + (int64_t)(rq_q0[rr] + rq) * q_stride + (int64_t)rh * D + c * (16 / sizeof(T));
      const uint32_t dst = smem_u32(sQ) + swz<D>(BM, r, c);
      if (!rotated) {
        cp_async16(dst, src, ok);
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
        const int shift = rq_shift[rr];
        const TR* cr = rope_cos + (int64_t)shift * rope_stride;
        const TR* sr = rope_sin + (int64_t)shift * rope_stride;
        const int d = c * E;
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const float x1 = to_f32<T>(a.e[e]), x2 = to_f32<T>(bb.e[e]);
          o1.e[e] = from_f32<T>(rot_lo<TC>(x1, x2, to_f32<TR>(cr[d + e]), -to_f32<TR>(sr[d + e])));
          o2.e[e] = from_f32<T>(rot_hi<TC>(x1, x2, to_f32<TR>(cr[d + D / 2 + e]), -to_f32<TR>(sr[d + D / 2 + e])));
        }
        *reinterpret_cast<uint4*>(sQ + swz<D>(BM, r, c)) = o1.u;
        *reinterpret_cast<uint4*>(sQ + swz<D>(BM, r, c + CH / 2)) = o2.u;
      }
    }
  };
  // keys [j0, j_end) of the tile's run; rr = the one request of the item the tile belongs to, -1 = all
  auto tile_span = [&](int i, int& j0, int& j_end, int& rr) {
    if (i < nt0) {
      j0 = i * BN;
      j_end = n_shared;
      rr = -1;
      return;
    }
    rr = 0;
    if (SPLIT) {
#pragma unroll
      for (int r = 1; r < GROUP; ++r)
        if (i >= t0r[r]) rr = r;
    }
    int first = nt0, len = kv_len;
#pragma unroll
    for (int r = 0; r < GROUP; ++r)
      if (r == rr) {
        first = t0r[r];
        len = klen[r];
      }
    j0 = n_shared + (i - first) * BN;
    j_end = len;
  };
  // ---- slot lookup -----------------------------------------------------------------------
  // Entry codes: >= 0 a slot, -1 a key that takes no part, -2 an entry outside the cache
  // (reported), -3 past the end of the run.  Lane l holds rows l and l + 32 of the tile.
  constexpr int ITER = BN * CH / NT;   // rows gathered per thread and tile
  constexpr int RPI = NT / CH;         // rows covered per iteration
  const int my_c = ltid % CH, my_r = ltid / CH;
  // The words of the slot map (or block table) are only LOADED here, two tiles ahead, and not
  // looked at before the end of the iteration, so no warp waits for them.
  constexpr int NR = GR;                  // requests whose entries a warp reads
  auto fetch_raw = [&](int i, int32_t (&raw)[NR][2]) {
    int j0, j_end, rr;
    tile_span(i, j0, j_end, rr);
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      const int first = (SPLIT && kind_a) ? rq_kv0[r] : kv0;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int j = j0 + h * 32 + lane;
        int32_t v = 0;
        if (j < j_end && r < n_req && (rr < 0 || rr == r))
          v = slot_map ? slot_map[first + j] : block_tables[(int64_t)b * table_stride + j / block_size];
        raw[r][h] = v;
      }
    }
  };
  // e0/e1: the entries the rows are fetched from (grouped: the union over the item's requests);
  // dead: the rows this warp's own request may not see
  auto interpret = [&](int i, const int32_t (&raw)[NR][2], int32_t& e0, int32_t& e1, uint32_t& dead_lo,
                       uint32_t& dead_hi) {
    int j0, j_end, rr;
    tile_span(i, j0, j_end, rr);
    int32_t uni[2] = {-3, -3}, own[2] = {-3, -3};
    bool clash = false;
    // the request whose view of the tile this warp works out (a group: one request per warp)
    const int own_r = (SPLIT && kind_a) ? ((LOADERS ? warp - 5 : warp) & 3) / CP : 0;
#pragma unroll
    for (int r = 0; r < NR; ++r) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int j = j0 + h * 32 + lane;
        int32_t code = -3;
        if (j < j_end && r < n_req && (rr < 0 || rr == r)) {
          int64_t slot = raw[r][h];
          if (slot_map) {
            code = slot == -1 ? -1 : ((slot < 0 || slot >= num_slots) ? -2 : (int32_t)slot);
          } else {
            slot = slot < 0 ? -2 : slot * block_size + j % block_size;
            code = (slot < 0 || slot >= num_slots) ? -2 : (int32_t)slot;  // fits 32 bits: the dispatcher refuses larger caches
          }
        }
        clash |= code >= 0 && uni[h] >= 0 && code != uni[h];
        uni[h] = max(uni[h], code);
        if (r == own_r) own[h] = code;
      }
    }
    e0 = uni[0];
    e1 = uni[1];
    dead_lo = __ballot_sync(0xFFFFFFFFu, own[0] < 0);
    dead_hi = __ballot_sync(0xFFFFFFFFu, own[1] < 0);
    if (err_flag) {
      if (clash) atomicExch(err_flag, 7);  // grouping contract: one span for the whole group
      if (uni[0] == -2 || uni[1] == -2) atomicExch(err_flag, 3);
    }
  };
  auto load_rows = [&](int i, int32_t e0, int32_t e1, const bool want_k, const bool want_v) {
    const uint32_t kb = smem_u32(sK) + (i & 1) * KV_BYTES, vb = smem_u32(sV) + (i & 1) * KV_BYTES;
    int j0, j_end, rr_unused;
    tile_span(i, j0, j_end, rr_unused);
    const int c = my_c;
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      const int r = my_r + it * RPI;
      const int j = j0 + r;
      int64_t slot = __shfl_sync(0xFFFFFFFFu, (it * RPI < 32) ? e0 : e1, r & 31);
      const bool ok = slot >= 0;
      if (!ok) slot = 0;
      const int64_t off = slot * kv_row + (int64_t)kvh * D + c * (16 / sizeof(T));
      const uint32_t so = swz<D>(BN, r, c);
      if (want_v) cp_async16(vb + so, v_cache + off, ok);
      if (!want_k) continue;
      if (!KEYSIDE) {
        cp_async16(kb + so, k_cache + off, ok);
      } else if (c < CH / 2) {
        // key-side relocation: a key that lives in the shared span is rotated by the table row
        // |j - slot| (sine negated when j < slot), rounded to T, before it is staged
        constexpr int E = 16 / sizeof(T);
        Vec16<T> a, bb;
        a.u = make_uint4(0, 0, 0, 0);
        bb.u = a.u;
        if (ok) {
          a.u = *reinterpret_cast<const uint4*>(k_cache + off);
          bb.u = *reinterpret_cast<const uint4*>(k_cache + off + D / 2);
          if (slot < shared_prefix_len) {
            const int64_t delta = (int64_t)j - slot;
            const bool neg = delta < 0;
            const int64_t row = neg ? -delta : delta;
            if (row >= rope_rows) {
              if (err_flag) atomicExch(err_flag, 4);
            } else {
              const TR* cr = rope_cos + row * rope_stride;
              const TR* sr = rope_sin + row * rope_stride;
              const int d = c * E;
#pragma unroll
              for (int e = 0; e < E; ++e) {
                const float x1 = to_f32<T>(a.e[e]), x2 = to_f32<T>(bb.e[e]);
                float s1 = to_f32<TR>(sr[d + e]), s2 = to_f32<TR>(sr[d + D / 2 + e]);
                if (neg) { s1 = -s1; s2 = -s2; }
                a.e[e] = from_f32<T>(rot_lo<TC>(x1, x2, to_f32<TR>(cr[d + e]), s1));
                bb.e[e] = from_f32<T>(rot_hi<TC>(x1, x2, to_f32<TR>(cr[d + D / 2 + e]), s2));
              }
            }
          }
        }
        *reinterpret_cast<uint4*>(sK + (i & 1) * KV_BYTES + so) = a.u;
        *reinterpret_cast<uint4*>(sK + (i & 1) * KV_BYTES + swz<D>(BN, r, c + CH / 2)) = bb.u;
      }
    }
  };

  const uint32_t idesc_s = make_idesc(Fmt<T>::id, 0, BN, BM);
  const uint32_t idesc_o = make_idesc(Fmt<T>::id, 1, D, BM);

  // a warp is live when at least one of its 32 rows is a real (query, head) pair
  const bool warp_live = (kind_a || spread) ? my_vrows > 0 : m0 + warp * 32 < my_vrows;
  float m_ref = -INFINITY, l_sum = 0.f;
  bool failed = false;

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
  // P V(t) done: barrier t & 1 of the pair, its (t >> 1)-th completion.  Two barriers, because a
  // row-owning warp no longer waits for every product: a parity wait is only right while the
  // barrier is at most one phase past the awaited one, and with one barrier for all tiles a warp
  // that is late for its wait for P V(t) could find P V(t+1) done as well and wait for ever.
  // With two, the phase before the awaited one (P V(t-2)) is over whenever S(t+1) or P V(t-1) has
  // been seen, and the phase after it (P V(t+2)) needs this thread's P(t+2)
  auto wait_pv = [&](int t) { return wait_bar(bar_o + (t & 1) * 8, (uint32_t)((t >> 1) & 1)); };
  // barrier of the 128 row-owning threads only (warp 4 never takes part)
  auto rows_sync = [&]() { asm volatile("bar.sync 1, 128;" ::: "memory"); };

  uint32_t dead_lo = 0, dead_hi = 0;   // rows of the current tile that take no part
  // online softmax of this thread's row over NC key columns of the tile starting at col0, exp2
  // domain; raw scores are scaled inside the fma.  First half: scores and their maximum.
  uint32_t s[BN];
  float mx;
  bool grow;
  bool pv_ok = true;   // false when the wait for a P V product inside the softmax ran out
  auto softmax_scores = [&](auto nc_tag, const int col0, const int i) {
    constexpr int NC = decltype(nc_tag)::value;
    if constexpr (NC == 64) {
      tmem_ld32(t_lane + kColS + (i & 1) * BN, s);
      tmem_ld32(t_lane + kColS + (i & 1) * BN + 32, s + 32);
    } else if constexpr (NC == 32) {
      tmem_ld32(t_lane + kColS + (i & 1) * BN + col0, s);
    } else {
      static_assert(NC == 16, "column slices are 16, 32 or 64 wide");
      tmem_ld16(t_lane + kColS + (i & 1) * BN + col0, s);
    }
    tmem_wait_ld();
    const uint64_t dead = ((((uint64_t)dead_hi) << 32) | dead_lo) >> col0;
    mx = -INFINITY;
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const float v = ((dead >> c) & 1ull) ? -INFINITY : __uint_as_float(s[c]);
      s[c] = __float_as_uint(v);
      mx = fmaxf(mx, v);
    }
    mx *= scale_log2;
    grow = mx > m_ref + 8.0f;  // also true on the first tile with a live key (m_ref = -inf)
  };
  // Second half, once the previous P V product is done: lazy rescale of O, P
  auto softmax_weights = [&](auto nc_tag, const int col0, const int i) {
    constexpr int NC = decltype(nc_tag)::value;
    if (__any_sync(0xFFFFFFFFu, grow) && i > 0) {
      // O may only be touched between two products: P V(i-1) done (the scores of tile i have been
      // seen, so P V(i-2) and everything before it is), and P V(i) is not issued before this thread
      // publishes P(i)
      pv_ok = wait_pv(i - 1) && pv_ok;
      tc_fence_after();
      const float f = grow ? ex2(m_ref - mx) : 1.0f;
      l_sum *= f;
      uint32_t o[32];
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        tmem_ld32(t_lane + kColO + c0, o);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * f);
        tmem_st32(t_lane + kColO + c0, o);
      }
      tmem_wait_st();
    }
    if (grow) m_ref = mx;
    const float m_use = m_ref == -INFINITY ? 0.f : m_ref;   // no live key so far: every p is 0
    float rs = 0.f;
    uint32_t w[NC / 2];   // this thread's weights, two per word
#pragma unroll
    for (int c = 0; c < NC; c += 2) {
      const float p0 = ex2(fmaf(__uint_as_float(s[c]), scale_log2, -m_use));
      const float p1 = ex2(fmaf(__uint_as_float(s[c + 1]), scale_log2, -m_use));
      rs += p0 + p1;
      w[c / 2] = pack2<T>(p0, p1);
    }
    // P(i) takes the place of the first 32 columns of S buffer i & 1 in TMEM (two weights per
    // column), where the P V product reads it as its A operand; a thread that runs the softmax of
    // a slice of the columns only writes zeros over the rest of its row
    const uint32_t p_at = t_lane + kColS + (i & 1) * BN;
    if constexpr (NC == 64) {
      tmem_st32(p_at, w);
    } else if constexpr (NC == 32) {
      if (col0 == 0) {
        tmem_st16(p_at, w);
        tmem_fill16(p_at + 16, 0u);
      } else {
        tmem_fill16(p_at, 0u);
        tmem_st16(p_at + 16, w);
      }
    } else {
#pragma unroll
      for (int gq = 0; gq < 4; ++gq) {
        if (gq * 16 == col0) tmem_st8(p_at + gq * 8, w);
        else tmem_fill8(p_at + gq * 8, 0u);
      }
    }
    tmem_wait_st();
    l_sum += rs;
  };
  auto softmax_half = [&](const bool second, const int i) {
    if (!warp_live) return;  // warps whose 32 rows are all padding skip the softmax (their P rows stay zero)
    if (SPLIT && dead_lo == 0xFFFFFFFFu && dead_hi == 0xFFFFFFFFu) {
      // a tile of another request of the group: no key of it counts for these rows
      if (second) {
        tmem_fill16(t_lane + kColS + (i & 1) * BN, 0u);
        tmem_fill16(t_lane + kColS + (i & 1) * BN + 16, 0u);
        tmem_wait_st();
      }
      return;
    }
    if constexpr (CP > 1) {
      if (!second) softmax_scores(std::integral_constant<int, BN / CP>{}, ci * (BN / CP), i);
      else softmax_weights(std::integral_constant<int, BN / CP>{}, ci * (BN / CP), i);
      return;
    }
    if (!second) softmax_scores(std::integral_constant<int, BN>{}, 0, i);
    else softmax_weights(std::integral_constant<int, BN>{}, 0, i);
  };

  // Roles.  Warp 4, one thread: issues S(i+1) as soon as K(i+1) has landed, i.e. one tile
  // ahead of the softmax (two S buffers in TMEM), and P V(i) as soon as P(i) is written.
  // Warps 0-3: stage K/V, run the softmax, never wait for one another inside the loop, only
  // for the products they consume.  In iteration i a row-owning thread
  //   publishes K(i+1) (its copies have landed)                        -> bar_k
  //   waits for S(i); K(i+2) may then overwrite K(i)
  //   waits for P V(i-1); V(i+1) may then overwrite V(i-1), O may be rescaled, P overwritten
  //   writes P(i) and publishes it together with V(i) having landed     -> bar_p
  // cp.async groups are committed in the fixed order K(i+2), V(i+1) per iteration (prologue:
  // Q+K(0), K(1), V(0)), so "one group pending" means K(i+1) has landed at the top of an
  // iteration and "two groups pending" means V(i) has landed at its end.
  if (warp == 4) {
    if (lane == 0 && n_tiles > 0) {
      auto issue_s = [&](int i) {   // S(i) = Q K(i)^T into S buffer i & 1
        const uint32_t kb = smem_u32(sK) + (i & 1) * KV_BYTES;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t a_off = (ks / 4) * (BM * 128) + (ks % 4) * 32;
          const uint32_t b_off = (ks / 4) * (BN * 128) + (ks % 4) * 32;
          mma_ss(tmem_base + kColS + (i & 1) * BN, make_desc(smem_u32(sQ) + a_off, 16, 1024),
                 make_desc(kb + b_off, 16, 1024), idesc_s, ks > 0 ? 1u : 0u);
        }
        mma_commit(bar_s + (i & 1) * 8);
      };
      bool ok = wait_bar(bar_k, 0);
      tc_fence_after();
      if (LOADERS) __threadfence_block();
      if (ok) issue_s(0);
      for (int i = 0; i < n_tiles && ok; ++i) {
        if (i + 1 < n_tiles) {
          // S buffer (i+1)&1 held S(i-1), read before P(i-1) was published, which was awaited
          ok = wait_bar(bar_k + ((i + 1) & 1) * 8, (uint32_t)(((i + 1) >> 1) & 1));
          tc_fence_after();
          if (!ok) break;
          if (LOADERS) __threadfence_block();   // what the loaders wrote before K(i+1) (the tile's dead rows) is passed on
          issue_s(i + 1);
        }
        ok = wait_bar(bar_p + (i & 1) * 8, (uint32_t)((i >> 1) & 1));
        if (LOADERS) ok = wait_bar(bar_v + (i & 1) * 8, (uint32_t)((i >> 1) & 1)) && ok;
        tc_fence_after();
        if (!ok) break;
        const uint32_t vb = smem_u32(sV) + (i & 1) * KV_BYTES;
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks) {
          mma_ts(tmem_base + kColO, tmem_base + kColS + (i & 1) * BN + ks * 8, make_desc(vb + ks * 2048, BN * 128, 1024),
                 idesc_o, (i > 0 || ks > 0) ? 1u : 0u);
        }
        mma_commit(bar_o + (i & 1) * 8);
      }
    }
  } else if (n_tiles > 0 && (!LOADERS || is_loader)) {
    // ---- the threads that stage K/V (and, without loader warps, also own the rows) ---------
    // every loader warp publishes the mask of the request it looks at (all the same unless a group)
    auto publish_dead = [&](int tile, uint32_t lo, uint32_t hi) {
      if (LOADERS && lane == 0) {
        dead_ring[((tile & 3) * 4 + ((warp - 5) & 3)) * 2] = lo;
        dead_ring[((tile & 3) * 4 + ((warp - 5) & 3)) * 2 + 1] = hi;
      }
    };
    const bool start_rotated = query_side && nt0 > 0;
    int32_t raw[NR][2];
    int32_t ev0 = -3, ev1 = -3, ek0 = -3, ek1 = -3;        // entries of tile i+1 (V load) / tile i+2 (K load)
    uint32_t dead1_lo = 0, dead1_hi = 0, dead2_lo = 0, dead2_hi = 0;  // tiles i+1, i+2 (dead_lo/hi: tile i)
    {
      int32_t raw0[NR][2], e0, e1;
      fetch_raw(0, raw0);                        // the lookups of the first tiles and the query tile
      if (n_tiles > 1) fetch_raw(1, raw);        // are all in flight before anything is read
      load_q(start_rotated);
      interpret(0, raw0, e0, e1, dead_lo, dead_hi);
      load_rows(0, e0, e1, true, false);
      cp_async_commit();                                   // Q + K(0)
      if (n_tiles > 1) {
        interpret(1, raw, ev0, ev1, dead1_lo, dead1_hi);
        load_rows(1, ev0, ev1, true, false);
      }
      cp_async_commit();                                   // K(1)
      load_rows(0, e0, e1, false, true);
      cp_async_commit();                                   // V(0)
      if (n_tiles > 2) {
        fetch_raw(2, raw);
        interpret(2, raw, ek0, ek1, dead2_lo, dead2_hi);
      }
      publish_dead(0, dead_lo, dead_hi);
      publish_dead(1, dead1_lo, dead1_hi);
      publish_dead(2, dead2_lo, dead2_hi);
    }
    cp_async_wait<2>();            // Q + K(0)
    fence_proxy_async();
    arrive(bar_k);

    bool ok = true;
    for (int i = 0; i < n_tiles; ++i) {
      if (i + 3 < n_tiles) fetch_raw(i + 3, raw);   // looked at when the iteration ends
      // query tile swap at the partition boundary: S(i) was the last product against the
      // rotated queries; S(i+1) may only be issued after the plain ones are in place
      if (start_rotated && i + 1 == nt0 && nt1 > 0) {
        ok = wait_bar(bar_s + (i & 1) * 8, (uint32_t)((i >> 1) & 1)) && ok;
        load_q(false);
        cp_async_commit();
        cp_async_wait<0>();
      }
      if (i + 1 < n_tiles) {
        cp_async_wait<1>();                            // K(i+1) has landed for this thread
        fence_proxy_async();
        arrive(bar_k + ((i + 1) & 1) * 8);
      }
      ok = wait_bar(bar_s + (i & 1) * 8, (uint32_t)((i >> 1) & 1)) && ok;
      tc_fence_after();
      if (i + 2 < n_tiles) load_rows(i + 2, ek0, ek1, true, false);   // S(i) is done: K(i) may go
      cp_async_commit();                               // K(i+2)
      if (!LOADERS) softmax_half(false, i);
      // the previous P V product must be done before O is rescaled, P overwritten or its V
      // stage refilled
      if (i > 0) ok = wait_pv(i - 1) && ok;
      tc_fence_after();
      if (i + 1 < n_tiles) load_rows(i + 1, ev0, ev1, false, true);
      cp_async_commit();                               // V(i+1)
      if (!LOADERS) softmax_half(true, i);
      cp_async_wait<2>();                              // V(i) has landed for this thread
      fence_proxy_async();
      tc_fence_before();
      if (LOADERS) arrive(bar_v + (i & 1) * 8);
      else arrive(bar_p + (i & 1) * 8);
      dead_lo = dead1_lo;
      dead_hi = dead1_hi;
      dead1_lo = dead2_lo;
      dead1_hi = dead2_hi;
      ev0 = ek0;
      ev1 = ek1;
      if (i + 3 < n_tiles) {
        interpret(i + 3, raw, ek0, ek1, dead2_lo, dead2_hi);
        // ring slot (i+3)&3 held tile i-1, whose softmax ended before P V(i-1) was issued
        publish_dead(i + 3, dead2_lo, dead2_hi);
      }
      if (!ok) break;
    }
    if (!LOADERS) {
      if (ok) ok = wait_pv(n_tiles - 1);
      tc_fence_after();
      if (!ok) *give_up = 1;
      rows_sync();
      failed = *give_up != 0;
    } else if (!ok) {
      *give_up = 1;
    }
  } else if (n_tiles > 0) {
    // ---- row-owning warps when loader warps do the staging: softmax only ----------------------
    // (rows of padding need no P: their queries are zero, so are their scores, and a zero score
    // reads as a zero weight)
    bool ok = true;
    for (int i = 0; i < n_tiles; ++i) {
      ok = wait_bar(bar_s + (i & 1) * 8, (uint32_t)((i >> 1) & 1)) && ok;   // also: the tile's dead rows are published
      tc_fence_after();
      dead_lo = dead_ring[((i & 3) * 4 + warp) * 2];
      dead_hi = dead_ring[((i & 3) * 4 + warp) * 2 + 1];
      // no wait for the previous P V product: P(i) lives in the S buffer it came from, and the
      // rescale of O, when a maximum moves, waits for it itself
      softmax_half(false, i);
      softmax_half(true, i);
      ok = ok && pv_ok;
      tc_fence_before();
      arrive(bar_p + (i & 1) * 8);
      if (!ok) break;
    }
    if (ok) ok = wait_pv(n_tiles - 1);
    tc_fence_after();
    if (!ok) *give_up = 1;
    rows_sync();
    failed = *give_up != 0;
  }

  if (warp >= 4) {
    // nothing to write
  } else if (failed) {
    if (tid == 0 && err_flag) atomicExch(err_flag, 5);
  } else if (CP > 1) {
    // ---- fold the column slices (copies) of every row, then write the rows -----------------------
    constexpr int F4 = D / 4;                       // float4 per row
    cp_async_wait<0>();
    float* xm = reinterpret_cast<float*>(sQ);       // [128] reference maxima, [128] row sums (the queries are no longer read)
    float4* part = reinterpret_cast<float4*>(sK);   // [4 warps][32 rows][F4], float4 index swizzled by the row
    xm[tid] = m_ref;
    xm[BM + tid] = l_sum;
    rows_sync();
    // copies of request slot rs sit in warps rs * CP .. rs * CP + CP - 1; same order for every reader
    auto fold_ml = [&](int rs, int row, float& m_all, float& l_all) {
      m_all = -INFINITY;
#pragma unroll
      for (int c = 0; c < CP; ++c) m_all = fmaxf(m_all, xm[(rs * CP + c) * 32 + row]);
      l_all = 0.f;
#pragma unroll
      for (int c = 0; c < CP; ++c) {
        const float mc = xm[(rs * CP + c) * 32 + row];
        l_all += mc == -INFINITY ? 0.f : xm[BM + (rs * CP + c) * 32 + row] * ex2(mc - m_all);
      }
    };
    float m_all, l_all;
    fold_ml(ri, lane, m_all, l_all);
    const float w_own = m_ref == -INFINITY ? 0.f : ex2(m_ref - m_all);
    const bool have = n_tiles > 0;                  // otherwise O was never written: it counts as 0
    uint32_t o[32];
#pragma unroll 1
    for (int c0 = 0; c0 < D; c0 += 32) {
      if (have) {
        tmem_ld32(t_lane + kColO + c0, o);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c) o[c] = 0u;
      }
#pragma unroll
      for (int c = 0; c < 32; c += 4) {
        const int idx = (c0 + c) / 4;
        part[(warp * 32 + lane) * F4 + (idx ^ (lane & (F4 - 1)))] =
            make_float4(__uint_as_float(o[c]) * w_own, __uint_as_float(o[c + 1]) * w_own,
                        __uint_as_float(o[c + 2]) * w_own, __uint_as_float(o[c + 3]) * w_own);
      }
    }
    rows_sync();
    // the item has GR x 32 output rows; TPR threads share one, each a 1 / TPR part of its columns
    constexpr int TPR = NT / (GR * 32);
    const int orow = tid / TPR, pt = tid % TPR;
    const int rs = orow >> 5, r = orow & 31;
    constexpr int QF4 = F4 / TPR;                   // float4 per thread
    float4 acc[QF4];
#pragma unroll
    for (int k = 0; k < QF4; ++k) {
      const int idx = pt * QF4 + k;
      float4 a4 = part[((rs * CP) * 32 + r) * F4 + (idx ^ (r & (F4 - 1)))];
#pragma unroll
      for (int c = 1; c < CP; ++c) {
        const float4 b4 = part[((rs * CP + c) * 32 + r) * F4 + (idx ^ (r & (F4 - 1)))];
        a4.x += b4.x; a4.y += b4.y; a4.z += b4.z; a4.w += b4.w;
      }
      acc[k] = a4;
    }
    fold_ml(rs, r, m_all, l_all);
    const bool r_ok = r < rq_vrows[rs];
    const int r_qi = r_ok ? r / g : 0, r_head = kvh * g + (r_ok ? r % g : 0);
    const int64_t r_qrow = (int64_t)rq_q0[rs] + r_qi;
    T* r_out = out + r_qrow * o_stride + (int64_t)r_head * D + pt * (D / TPR);
    const float a_own = l_all > 0.f ? 1.0f / l_all : 0.f;
    if (r_ok) {
#pragma unroll
      for (int k = 0; k < QF4; k += 2) {
        const float4 x0 = acc[k], x1 = acc[k + 1];
        uint4 w;
        w.x = pack2<T>(x0.x * a_own, x0.y * a_own);
        w.y = pack2<T>(x0.z * a_own, x0.w * a_own);
        w.z = pack2<T>(x1.x * a_own, x1.y * a_own);
        w.w = pack2<T>(x1.z * a_own, x1.w * a_own);
        *reinterpret_cast<uint4*>(r_out + k * 4) = w;
      }
    }
  } else {
    // thread = row: divide by the row sum and write (a group: warp w writes request w's rows)
    const float inv = l_sum > 0.f ? 1.0f / l_sum : 0.f;
    uint32_t o[32];
#pragma unroll 1
    for (int c0 = 0; c0 < D; c0 += 32) {
      tmem_ld32(t_lane + kColO + c0, o);
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
  cp_async_wait<0>();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

template <typename T, typename TR> struct PromoteT { using type = float; };
template <> struct PromoteT<__half, __half> { using type = __half; };
template <> struct PromoteT<__nv_bfloat16, __nv_bfloat16> { using type = __nv_bfloat16; };

template <typename T, typename TR, int D>
static int launch(const AttnArgs& a, const SplitArgs* split) {
  using TC = typename PromoteT<T, TR>::type;
  constexpr size_t smem = BM * D * sizeof(T) + 4 * BN * D * sizeof(T) + 512;
  const int g = a.n_heads / a.n_kv_heads;
  const bool relocate = a.shared_prefix_len > 0 && a.affix_shifts != nullptr;
  const bool query_side = relocate && a.shared_kv_lens != nullptr;
  const bool key_side = relocate && !query_side;
  SplitArgs sp{};
  dim3 grid((a.max_q * g + BM - 1) / BM, a.batch, a.n_kv_heads);
  if (split) {
    sp = *split;
    grid = dim3(sp.n_items_a, 1, 1);
  }
#define ACACHE_TC_LAUNCH(KS, SPL, CP, LD)                                                                             \
  do {                                                                                                                \
    auto kern = attention_tc_kernel<T, TR, TC, D, KS, SPL, CP, LD>;                                                   \
    ACACHE_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));            \
    ACACHE_CUDA_CHECK(launch_chained(                                                                                 \
        kern, grid, dim3(LD ? NT_LOAD : NT_ALL), smem, a.st,                                                          \
        (const T*)a.q, a.q_stride, (T*)a.out, a.o_stride, (const T*)a.k_cache, (const T*)a.v_cache, a.num_slots,      \
        a.n_heads, a.n_kv_heads, a.cu_q, a.cu_k, a.slot_map, a.block_tables, a.table_stride, a.block_size,            \
        a.scale * 1.4426950408889634f, a.shared_prefix_len, a.shared_kv_lens,                                         \
        relocate ? a.affix_shifts : (const int32_t*)nullptr, (const TR*)a.rope_cos, (const TR*)a.rope_sin,            \
        a.rope_stride, a.rope_rows, a.err_flag, sp));                                                                 \
  } while (0)
  // requests of at most 32 virtual rows (block decode): spread the softmax over the four warps
  // and give the K/V staging to four more warps
  const bool small_rows = a.max_q * g <= 32;
  if (split) ACACHE_TC_LAUNCH(false, true, 2, true);
  else if (key_side) ACACHE_TC_LAUNCH(true, false, 1, false);
  else if (small_rows) ACACHE_TC_LAUNCH(false, false, 4, true);
  else ACACHE_TC_LAUNCH(false, false, 1, false);
#undef ACACHE_TC_LAUNCH
  ACACHE_LAUNCH_CHECK();
  return ACACHE_OK;
}

template <typename T, typename TR>
static int by_dim(const AttnArgs& a, const SplitArgs* split) {
  if (a.head_dim == 128) return launch<T, TR, 128>(a, split);
  if (a.head_dim == 64) return launch<T, TR, 64>(a, split);
  return ACACHE_EUNSUPPORTED;
}

static int by_dtype(const AttnArgs& a, int dtype, int rope_dtype, const SplitArgs* split) {
  if (dtype == ACACHE_F32 || a.num_slots >= (1ll << 31)) return ACACHE_EUNSUPPORTED;
  if (a.head_dim != 64 && a.head_dim != 128) return ACACHE_EUNSUPPORTED;
  if (!aligned16(a.q) || !aligned16(a.out) || !aligned16(a.k_cache) || !aligned16(a.v_cache)) return ACACHE_EUNSUPPORTED;
  if (a.q_stride % 8 != 0 || a.o_stride % 8 != 0) return ACACHE_EUNSUPPORTED;
  if (split == nullptr) {
    const int rc = attention_tc256_dispatch(a, dtype, rope_dtype);
    if (rc != ACACHE_EUNSUPPORTED) return rc;
  }
  if (dtype == ACACHE_BF16) {
    if (rope_dtype == ACACHE_F32) return by_dim<__nv_bfloat16, float>(a, split);
    if (rope_dtype == ACACHE_BF16) return by_dim<__nv_bfloat16, __nv_bfloat16>(a, split);
    return by_dim<__nv_bfloat16, __half>(a, split);
  }
  if (rope_dtype == ACACHE_F32) return by_dim<__half, float>(a, split);
  if (rope_dtype == ACACHE_F16) return by_dim<__half, __half>(a, split);
  return by_dim<__half, __nv_bfloat16>(a, split);
}

}  // namespace tc

// Declines (ACACHE_EUNSUPPORTED) what this kernel does not cover: fp32 caches, head sizes
// other than 64/128, unaligned tensors.
int attention_tc_dispatch(const AttnArgs& a, int dtype, int rope_dtype) {
  return tc::by_dtype(a, dtype, rope_dtype, nullptr);
}

// The grouped form keeps nothing between its CTAs and needs no scratch.
int64_t attention_split_scratch_bytes(int total_q, int n_heads, int head_dim, int batch, int n_kv_heads) {
  (void)total_q; (void)n_heads; (void)head_dim; (void)batch; (void)n_kv_heads;
  return 0;
}

// Shared-span grouping; declines what it does not cover (also: relocation on the key side,
// block tables, more than 32 virtual rows per request, no shared_kv_lens).
int attention_split_dispatch(const AttnArgs& a, int dtype, int rope_dtype, int total_q, void* scratch,
                             int64_t scratch_bytes) {
  (void)total_q; (void)scratch; (void)scratch_bytes;
  if (!a.slot_map || !a.shared_kv_lens) return ACACHE_EUNSUPPORTED;
  if (a.n_kv_heads <= 0 || a.n_heads % a.n_kv_heads != 0) return ACACHE_EINVAL;
  if (a.max_q * (a.n_heads / a.n_kv_heads) > 32) return ACACHE_EUNSUPPORTED;
  tc::SplitArgs sp;
  sp.n_items_a = ((a.batch + tc::kGroupedRequests - 1) / tc::kGroupedRequests) * a.n_kv_heads;
  sp.batch = a.batch;
  return tc::by_dtype(a, dtype, rope_dtype, &sp);
}

}  // namespace acache

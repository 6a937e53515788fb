// Vocabulary shards that exchange their candidates over peer memory.  Included inside namespace
// leat by sampler_kernels.cuh (the types ahead of KParams, the kernels after finish_list.cuh).
//
// Every rank owns a contiguous slice of the vocabulary (a tensor-parallel lm_head's layout) and a
// contiguous share of the rows.  A step on a rank:
//
//   filter_kernel        streams the rank's slice of every row once and lists what reaches each
//                        row's floor, as on one GPU
//   shard_select_kernel  one block per row: the listed logits penalised and scaled, the slice's
//                        candidates for the row (everything at or above its top_k-th score) stored
//                        straight into the exchange region of the rank that owns the row, over
//                        NVLink; the block that hands an owner its last row raises the owner's flag
//   sample_kernel        streams the rows the lists could not settle (usually none) and hands them
//                        over the same way
//   shard_finish_kernel  one block per owned row: waits (bounded) for every rank's flag, merges the
//                        slices' candidates, finishes the row, and stores the result into every
//                        rank's region; the last block raises this owner's flag everywhere
//   shard_result_kernel  waits (bounded) for every owner's flag and copies the results out
//
// Peer memory is only ever written (plain stores to peer-mapped addresses) and every rank reads its
// own region; no load crosses NVLink.  Flags carry the step's number, and every buffer exists twice
// (step parity), so nothing has to be cleared between steps: a rank can be at most one step ahead
// of any other, because it cannot end a step without every other rank's results.  Ranks must take
// the same steps in the same order.  A wait that runs out sets LEAT_STATUS_PEER in the status word
// and the step's ids read -1; no kernel spins without a limit.
//
// (Included twice: no include guard for the file as a whole.)

#ifndef LEAT_SHARD_TYPES
#define LEAT_SHARD_TYPES
constexpr int SHARD_MAX_WORLD = 8;
constexpr unsigned SHARD_WAIT_POLLS = 1u << 20;  // of about a microsecond each: a second or so

struct ShardView {
  unsigned char* region[SHARD_MAX_WORLD];  // every rank's exchange region, peer-mapped; [rank] is this rank's own
  int rank, world;
  int rows;   // rows of a step
  int owned;  // rows a rank owns: ceil(rows / world); rank r owns [r * owned, min(rows, (r + 1) * owned))
  int cap;    // candidates a rank may hand over per row
  unsigned* epoch;        // this rank's step number (starts at 1)
  unsigned* tickets;      // (world): rows handed to each owner so far this step
  unsigned* done_ticket;  // owned rows finished so far this step
  int* marks;             // (rows): -2 = the row is left to the streaming kernel
};

// a rank's hand-over for one row
struct ShardSlot {
  unsigned long long best;  // the slice's greedy key
  int count;                // candidates, or -1: the slice could not be reduced to `cap`
  int pad;
  unsigned long long keys[1];  // (cap) (score, id) keys, unordered
};
// a finished row, as every rank receives it
struct ShardResult {
  int id, greedy, kept;
  float cut;
};

__host__ __device__ inline size_t shard_slot_bytes(int cap) { return 16 + (size_t)cap * 8; }
__host__ __device__ inline size_t shard_round(size_t x) { return (x + 255) / 256 * 256; }
// region layout: slots [parity][source][local row] | arrive flags [parity][source] | results
// [parity][row] | done flags [parity][owner]
__host__ __device__ inline size_t shard_at_arrive(int world, int owned, int cap) {
  return shard_round((size_t)2 * world * owned * shard_slot_bytes(cap));
}
__host__ __device__ inline size_t shard_at_result(int world, int owned, int cap) {
  return shard_at_arrive(world, owned, cap) + shard_round((size_t)2 * world * 4);
}
__host__ __device__ inline size_t shard_at_done(int world, int owned, int cap) {
  return shard_at_result(world, owned, cap) + shard_round((size_t)2 * world * owned * sizeof(ShardResult));
}
__host__ __device__ inline size_t shard_region_bytes(int world, int owned, int cap) {
  return shard_at_done(world, owned, cap) + shard_round((size_t)2 * world * 4);
}
__device__ __forceinline__ void store_release_system(unsigned* at, unsigned value) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(at), "r"(value) : "memory");
}
__device__ __forceinline__ unsigned load_acquire_system(const unsigned* at) {
  unsigned value;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(value) : "l"(at) : "memory");
  return value;
}
// Polls a flag of this rank's own region until it carries `epoch`; false if it never does.
__device__ __forceinline__ bool shard_wait(const unsigned* flag, unsigned epoch) {
#pragma unroll 1
  for (unsigned poll = 0; poll < SHARD_WAIT_POLLS; ++poll) {
    if (load_acquire_system(flag) == epoch) return true;
    __nanosleep(200);
  }
  return false;
}

__device__ __forceinline__ ShardSlot* shard_slot(const ShardView& v, int owner, int parity, int source, int local) {
  return reinterpret_cast<ShardSlot*>(v.region[owner] +
                                      ((size_t)(parity * v.world + source) * v.owned + local) * shard_slot_bytes(v.cap));
}

// After a block has stored row `row`'s slot at its owner: the stores are made visible system-wide,
// the row is counted, and the block that counts the owner's last row raises the owner's flag.  The
// whole block calls it.
__device__ __forceinline__ void shard_hand_over(const ShardView& v, int row, unsigned epoch) {
  // The block's stores are ordered before thread 0's fence by the barrier, and before the ticket by
  // the fence; device scope is enough here, because the one block that goes on to raise the flag
  // fences at system scope after it has seen every other block's ticket (fences are cumulative).
  // A system fence per block was measured at about 10 us per 512 blocks.
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int owner = row / v.owned;
    const int theirs = min(v.owned, v.rows - owner * v.owned);
    const unsigned ticket = atomicAdd(&v.tickets[owner], 1u);
    if (ticket == (unsigned)(theirs - 1)) {
      v.tickets[owner] = 0u;
      __threadfence_system();
      unsigned* arrive = reinterpret_cast<unsigned*>(v.region[owner] + shard_at_arrive(v.world, v.owned, v.cap));
      store_release_system(&arrive[(epoch & 1u) * v.world + v.rank], epoch);
    }
  }
}
#endif  // LEAT_SHARD_TYPES

#ifdef LEAT_SHARD_KERNELS

// One block per row this rank owns: merges what every rank handed over for the row and finishes it.
template <int NT>
__global__ void __launch_bounds__(NT, 1024 / NT) shard_finish_kernel(const __grid_constant__ KParams P) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  FLShared& S = *reinterpret_cast<FLShared*>(smem_raw);
  unsigned* hist = reinterpret_cast<unsigned*>(smem_raw + FL_FIXED);
  unsigned long long* skeys = reinterpret_cast<unsigned long long*>(hist + FL_HIST_WORDS);
  unsigned* area = reinterpret_cast<unsigned*>(skeys + FL_KEYS);
  __shared__ int counts[SHARD_MAX_WORLD];
  __shared__ ShardResult result;
  const ShardView& v = P.shard;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int local = blockIdx.x, b = v.rank * v.owned + local;
  RowCfg& rc = S.rc;
  // ---- what needs no hand-over: the row's options, the histogram cleared ----
  if (warp == 0) {
    uint32_t unused;
    const RowIn in = row_inputs_warp(P, b, nullptr, unused);
    if (lane == 0) {
      rc = row_config_from(P, in);
      S.gbest = 0ull; S.best = 0ull; S.vmin = 0xFFFFFFFFu; S.vmax = 0u; S.rmin = 0xFFFFFFFFu; S.rmax = 0u;
      S.live = 0; S.m = 0; S.redo = 0;
      result.id = -1; result.greedy = -1; result.kept = 0; result.cut = quiet_nan();
    }
  }
  {
    uint4* h4 = reinterpret_cast<uint4*>(hist);
#pragma unroll 1
    for (int i = tid; i < BINS / 4; i += NT) h4[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  grid_dependency_wait();  // this rank's own hand-overs (and its step number) are settled
  stamp_begin(P.stamps, 4);
  const unsigned epoch = __ldcg(v.epoch);
  const int parity = (int)(epoch & 1u);
  // ---- every rank's flag, each polled by a thread of its own ----
  int arrived = 1;
  if (tid < v.world) {
    const unsigned* arrive = reinterpret_cast<const unsigned*>(v.region[v.rank] + shard_at_arrive(v.world, v.owned, v.cap));
    arrived = shard_wait(&arrive[parity * v.world + tid], epoch) ? 1 : 0;
    counts[tid] = arrived ? __ldcg(&shard_slot(v, v.rank, parity, tid, local)->count) : -1;
  }
  const bool all_here = __syncthreads_and(arrived) != 0;
  const int mode = rc.mode;
  bool failed = !all_here;
  int at[SHARD_MAX_WORLD + 1];
  at[0] = 0;
#pragma unroll
  for (int s = 0; s < SHARD_MAX_WORLD; ++s) {
    const int c = s < v.world ? counts[s] : 0;
    if (c < 0) failed = true;
    at[s + 1] = at[s] + max(c, 0);
  }
  const int n = at[SHARD_MAX_WORLD];
  if (!failed) {
    // ---- the slices' candidates side by side, and the row's greedy token ----
    unsigned long long gbest = 0ull;
    if (tid < v.world) gbest = __ldcg(&shard_slot(v, v.rank, parity, tid, local)->best);
    gbest = warp_max_u64(gbest);
    if (tid == 0) { S.gbest = gbest; result.greedy = key_id(gbest); }
    uint32_t mn = 0xFFFFFFFFu, mx = 0u;
    unsigned long long best = 0ull;
#pragma unroll 1
    for (int i = tid; i < n; i += NT) {
      int s = 0;
#pragma unroll
      for (int q = 1; q < SHARD_MAX_WORLD; ++q) s += i >= at[q] ? 1 : 0;
      const unsigned long long key = __ldcg(&shard_slot(v, v.rank, parity, s, local)->keys[i - at[s]]);
      skeys[i] = key;
      mx = max(mx, key_vbits(key));
      mn = min(mn, key_vbits(key));
      best = key > best ? key : best;
    }
    mx = __reduce_max_sync(FULL, mx);
    mn = __reduce_min_sync(FULL, mn);
    if (lane == 0 && mx >= mn) { atomicMax(&S.vmax, mx); atomicMin(&S.vmin, mn); }
    if (mode == M_ARGMAX_G) {  // whole-row hashed draw: every slice sent its best score + noise
      best = warp_max_u64(best);
      if (lane == 0) atomicMax(&S.best, best);
    }
    if (tid == 0) S.live = n;
  }
  __syncthreads();
  unsigned long long* cbuf = reinterpret_cast<unsigned long long*>(area);
  unsigned long long* runs = cbuf + FL_SORT;
  float* fw = reinterpret_cast<float*>(runs + FL_SORT);
  float* fx = fw + FL_SORT;
  float* fseg = fx + FL_SORT;
  if (!failed && (mode == M_SELECT_K || mode == M_SELECT_MINP)) {
    if (n == 0) {
      failed = true;
    } else {
      fl_select<NT>(skeys, n, rc.k_eff, mode == M_SELECT_MINP, rc.logm, hist, cbuf, S);
      const int c = S.m;
      if (c > FL_SORT) {
        failed = true;
      } else {
        fl_sort<NT>(cbuf, c, runs, cbuf);
        RowOut out;
        out.id = &result.id; out.cut = &result.cut; out.kept = &result.kept;
        out.probs = nullptr; out.prob_ids = nullptr; out.width = 0;
        fl_finish<NT, false>(P, rc, out, cbuf, c, S, fw, fx, fseg, neg_inf());
      }
    }
  } else if (!failed && tid == 0) {
    if (mode == M_ARGMAX_L) result.id = key_id(S.gbest);
    else if (mode == M_ARGMAX_G) { result.id = key_id(S.best); result.cut = neg_inf(); result.kept = P.vocab; }
    else failed = true;  // a row for the multi-pass routine: not taken by shards
  }
  __syncthreads();
  if (tid == 0 && (failed || mode == M_GENERAL) && P.status) atomicOr(P.status, all_here ? 4 : 12);
  // ---- the result to every rank; the last owned row raises this owner's flag everywhere ----
  if (tid < v.world) {
    ShardResult* dst = reinterpret_cast<ShardResult*>(v.region[tid] + shard_at_result(v.world, v.owned, v.cap)) +
                       (size_t)parity * v.world * v.owned + b;
    *reinterpret_cast<int4*>(dst) = *reinterpret_cast<const int4*>(&result);
  }
  __syncthreads();
  if (tid == 0) {
    __threadfence();  // (device scope: the last block fences at system scope below, as in shard_hand_over)
    const int mine = min(v.owned, v.rows - v.rank * v.owned);
    const unsigned ticket = atomicAdd(v.done_ticket, 1u);
    S.sel_bin = ticket == (unsigned)(mine - 1) ? 1 : 0;
    if (S.sel_bin) *v.done_ticket = 0u;
  }
  __syncthreads();
  if (S.sel_bin && tid < v.world) {
    __threadfence_system();
    unsigned* done = reinterpret_cast<unsigned*>(v.region[tid] + shard_at_done(v.world, v.owned, v.cap));
    store_release_system(&done[parity * v.world + v.rank], epoch);
  }
  stamp_end(P.stamps, 4);
}

// One block: waits for every owner's flag, copies the results out and ends the step.
__global__ void __launch_bounds__(256) shard_result_kernel(const __grid_constant__ KParams P) {
  const ShardView& v = P.shard;
  const int tid = threadIdx.x;
  grid_dependency_wait();
  stamp_begin(P.stamps, 5);
  const unsigned epoch = __ldcg(v.epoch);
  const int parity = (int)(epoch & 1u);
  int arrived = 1;
  if (tid < v.world) {
    // (a rank that owns no rows raises no flag)
    const unsigned* done = reinterpret_cast<const unsigned*>(v.region[v.rank] + shard_at_done(v.world, v.owned, v.cap));
    if (tid * v.owned < v.rows) arrived = shard_wait(&done[parity * v.world + tid], epoch) ? 1 : 0;
  }
  const bool all_here = __syncthreads_and(arrived) != 0;
  const ShardResult* results = reinterpret_cast<const ShardResult*>(v.region[v.rank] + shard_at_result(v.world, v.owned, v.cap)) +
                               (size_t)parity * v.world * v.owned;
#pragma unroll 1
  for (int b = tid; b < v.rows; b += blockDim.x) {
    int4 raw = __ldcg(reinterpret_cast<const int4*>(&results[b]));
    ShardResult r = *reinterpret_cast<ShardResult*>(&raw);
    if (!all_here) { r.id = -1; r.greedy = -1; r.kept = 0; r.cut = quiet_nan(); }
    if (P.out_ids) P.out_ids[b] = r.id;
    if (P.out_greedy) P.out_greedy[b] = r.greedy;
    if (P.out_kept) P.out_kept[b] = r.kept;
    if (P.out_cut) P.out_cut[b] = r.cut;
  }
  if (tid == 0) {
    if (!all_here && P.status) atomicOr(P.status, 12);
    *v.epoch = epoch + 1u;  // the step is over on this rank
  }
  stamp_end(P.stamps, 5);
}

#endif  // LEAT_SHARD_KERNELS

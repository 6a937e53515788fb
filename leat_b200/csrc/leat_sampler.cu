// Host side of libleat_sampler.so: argument checks, the launch plan, and the extern "C" entry
// points declared in include/leat_sampler.h.  Nothing here allocates device memory or synchronises
// after leat_sampler_create().
#include "../../include/leat_sampler.h"

#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <new>

#include "sampler_kernels.cuh"

using namespace leat;

namespace {

constexpr int kMaxSliceLen = 1 << 20;  // a block may take a whole row
constexpr int kSliceAlign = 128;
constexpr int kMaxK = 1024;
constexpr int kSpareCells = 4096;
constexpr int kArgmaxMinVocab = 4096;  // shorter rows go through the sampler's own greedy path
constexpr int kListCap = 4096;        // (logit, index) pairs a row's filter may list
constexpr int kFilterMinVocab = 16384;  // narrower rows are not worth three launches

thread_local char g_cuda_error[256] = "";

int cuda_failed(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return 0;
  snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s", what, cudaGetErrorString(e));
  return 1;
}

int round_up(int x, int m) { return (x + m - 1) / m * m; }
int next_pow2(int x) { int p = 1; while (p < x) p <<= 1; return p; }

struct Layout {
  size_t keys, count, best, vmin, ticket, flag, list, list_count, list_info, stamps, total;
  int cells;
};

Layout layout_for(int max_rows, int max_vocab, int keep) {
  Layout L;
  L.cells = max_rows * ((max_vocab + kMaxSliceLen - 1) / kMaxSliceLen) + kSpareCells;
  size_t at = 0;
  auto take = [&](size_t bytes) { size_t here = at; at += (bytes + 255) / 256 * 256; return here; };
  L.keys = take((size_t)L.cells * keep * 8);
  L.count = take((size_t)L.cells * 4);
  L.best = take((size_t)L.cells * 16);
  L.vmin = take((size_t)L.cells * 4);
  L.ticket = take((size_t)max_rows * 4);
  L.flag = take((size_t)max_rows * 4);
  L.list = take((size_t)max_rows * kListCap * 8);
  L.list_count = take((size_t)max_rows * 4);
  L.list_info = take((size_t)max_rows * 8);
  L.stamps = take(16 * 8);
  L.total = at;
  return L;
}

int keep_for(int k_max) { return round_up(k_max + 64, 64); }
int cap_for(int keep) { return keep <= 512 ? 2048 : 4096; }

}  // namespace

struct leat_sampler {
  int device, max_rows, max_vocab, k_max, keep, cap;
  int tune_threads, tune_slices, tune_no_filter, has_list;
  // optional per-kernel timing of a call: the kernels stamp their begin and end in the workspace
  int timing;
  // a launch failed after lists were written: the next call empties the lists first
  int dirty;
  int sm_count;
  int launches;
  unsigned char* ws;
  Layout L;
};

namespace {

struct Plan {
  int vec, threads, slices, slice_len, bm_words, ht_size, shared, ring_stages;
  int grid_rows;  // blocks along the grid's row axis: 0 = one per row, else each takes several rows in turn
};

constexpr int kMostShared = 200 * 1024;
constexpr size_t kFilterAhead = (size_t)FILTER_THREADS * FILTER_VECS * 16;  // one work item, on its way in while a floor is found  // dynamic shared memory the kernels are allowed

constexpr size_t kSharedPerBlockTarget = 112 * 1024;  // two blocks per SM

size_t fixed_shared(int cap, int keep) {
  return (size_t)cap * 8 + (size_t)keep * 8 + (size_t)(BINS + 32) * 4 + SMEM_FIXED;
}

size_t shared_bytes(int cap, int keep, int ht_size, size_t ring = 0) {
  // the hash keys, then one area shared by their counts, the ring and the scratch of the finish
  size_t keys = ((size_t)ht_size * 4 + 127) / 128 * 128;
  size_t counts = (size_t)ht_size * 8;  // counts and the tokens' logits
  size_t finish = (size_t)cap * 8 + (size_t)(cap / 16) * 4;  // weights, running sums, segment sums and offsets
  size_t later = counts > ring ? counts : ring;
  if (finish > later) later = finish;
  return fixed_shared(cap, keep) + keys + later;
}

Plan make_plan(const leat_sampler* h, int rows, int vocab, int history_cap, bool has_history, int vec) {
  Plan p;
  p.vec = vec;
  p.grid_rows = 0;
  p.threads = h->tune_threads ? h->tune_threads : 512;
  int step = p.threads * vec * UNROLL;
  int min_slices = (vocab + kMaxSliceLen - 1) / kMaxSliceLen;
  int max_slices = (vocab + step - 1) / step;
  if (max_slices < min_slices) max_slices = min_slices;
  // every block pays a fixed price (set-up, first threshold, final select), so rows are cut no
  // finer than it takes to give each of the two blocks an SM holds something to do
  int resident = h->sm_count * 2;
  int want = h->tune_slices ? h->tune_slices : (resident + rows / 2) / rows;
  if (!h->tune_slices && want > 8) want = 8;
  int by_cells = h->L.cells / (rows > 0 ? rows : 1);
  if (want > by_cells) want = by_cells;
  if (want > max_slices) want = max_slices;
  if (want < min_slices) want = min_slices;
  if (want < 1) want = 1;
  p.slice_len = round_up((vocab + want - 1) / want, kSliceAlign);
  if (p.slice_len < 1) p.slice_len = kSliceAlign;
  p.slices = (vocab + p.slice_len - 1) / p.slice_len;
  if (p.slices < 1) p.slices = 1;
  p.bm_words = 0;
  p.ht_size = has_history ? next_pow2(history_cap * 2 < 64 ? 64 : history_cap * 2) : 0;
  // the ring of bulk copies: as many stages as fit a block's share of shared memory
  p.ring_stages = 0;
  if (vec == 4) {
    const size_t stage = (size_t)p.threads * RING_PER_THREAD * 4;
    const size_t used = fixed_shared(h->cap, h->keep) + ((size_t)p.ht_size * 4 + 127) / 128 * 128;
    int stages = used < kSharedPerBlockTarget ? (int)((kSharedPerBlockTarget - used) / stage) : 0;
    if (stages > MAX_RING_STAGES) stages = MAX_RING_STAGES;
    if (stages >= 2) p.ring_stages = stages;
  }
  // the area behind the hash keys holds the ring, or at least a bitmap over the vocabulary (what a
  // listed row marks its history tokens in) when that is not large
  size_t behind = (size_t)p.ring_stages * p.threads * RING_PER_THREAD * 4;
  const size_t bitmap = has_history ? (size_t)(vocab + 31) / 32 * 4 : 0;
  if (bitmap <= 48 * 1024 && behind < bitmap) behind = bitmap;
  p.shared = (int)shared_bytes(h->cap, h->keep, p.ht_size, behind);
  // a row the single pass cannot settle is redone in place by the multi-pass routine, which lays
  // out the block's shared memory its own way
  const int redo = (int)(G_BINS * 12 + 384 + (size_t)p.ht_size * 8);
  if (p.shared < redo) p.shared = redo;
  // words of the area behind the hash keys: room for a bitmap over the vocabulary
  p.bm_words = (int)((p.shared - fixed_shared(h->cap, h->keep) - ((size_t)p.ht_size * 4 + 127) / 128 * 128) / 4);
  return p;
}

// finish_list_kernel's dynamic shared memory for a call, or 0 when the call's history is too long for
// it (then sample_kernel finishes listed rows too, as it does for shards).  ht: slots of its hash
// table; area_words: words behind its keys.
size_t lean_shared(int vocab, int history_cap, bool has_history, int old_ht_size, int* ht, int* area_words) {
  size_t area = (size_t)FL_AREA_MIN_WORDS * 4;
  *ht = 0;
  if (has_history) {
    *ht = next_pow2(history_cap * 2 < 64 ? 64 : history_cap * 2);
    const size_t table = (size_t)*ht * 8;
    if (table > 64 * 1024) return 0;
    if (table > area) area = table;
    const size_t bitmap = (size_t)(vocab + 31) / 32 * 4;
    if (bitmap <= 32 * 1024 && bitmap > area) area = bitmap;
  }
  area = (area + 15) / 16 * 16;
  *area_words = (int)(area / 4);
  size_t total = FL_FIXED + (size_t)FL_HIST_WORDS * 4 + (size_t)FL_KEYS * 8 + area;
  // a row the list cannot settle is redone in place by the multi-pass routine
  const size_t redo = G_BINS * 12 + 384 + (size_t)old_ht_size * 8;
  return total > redo ? total : redo;
}

bool aligned(const void* p, size_t a) { return ((uintptr_t)p % a) == 0; }

int check_broadcast(const void* p, int n, int rows) { return !p || n == rows || n == 1; }

int fill_params(const leat_sampler* h, const leat_sample_args* a, KParams& P) {
  if (!h || !a) return LEAT_E_ARGUMENT;
  if (a->rows < 0 || a->vocab <= 0) return LEAT_E_ARGUMENT;
  if (a->rows > h->max_rows || a->vocab > h->max_vocab) return LEAT_E_CAPACITY;
  if (a->rows == 0) {  // nothing to do, and nothing to point at
    memset(&P, 0, sizeof(P));
    P.vocab = a->vocab;
    return LEAT_OK;
  }
  if (!check_broadcast(a->options, a->options_rows, a->rows) ||
      !check_broadcast(a->seed, a->seed_rows, a->rows) ||
      !check_broadcast(a->position, a->position_rows, a->rows) ||
      !check_broadcast(a->penalties, a->penalties_rows, a->rows))
    return LEAT_E_ARGUMENT;
  if (a->history && a->history_cap <= 0) return LEAT_E_ARGUMENT;
  if (a->history && a->history_cap > 8192) return LEAT_E_CAPACITY;
  if ((a->out_probs || a->out_prob_ids) && a->out_width <= 0) return LEAT_E_ARGUMENT;
  memset(&P, 0, sizeof(P));
  P.logits = static_cast<const float*>(a->logits); P.rows = a->rows; P.vocab = a->vocab; P.row_stride = a->row_stride;
  P.vocab_total = a->vocab_total > 0 ? a->vocab_total : a->vocab;
  P.options = a->options; P.options_rows = a->options_rows;
  P.seed = a->seed; P.seed_rows = a->seed_rows;
  P.position = a->position; P.position_rows = a->position_rows;
  P.seen = a->seen; P.seen_stride = a->seen_stride;
  P.history = a->history; P.history_len = a->history_len; P.history_cap = a->history ? a->history_cap : 0;
  P.penalties = a->penalties; P.penalties_rows = a->penalties_rows;
  P.uniform = a->uniform;
  P.vocab_offset = a->vocab_offset; P.flags = a->flags;
  if (!(a->softcap >= 0.0f)) return LEAT_E_ARGUMENT;
  P.softcap = a->softcap; P.position_scalar = a->position_scalar;
  if ((a->flags & LEAT_FLAG_LOGITS_BF16) && (a->flags & LEAT_FLAG_LOGITS_F16)) return LEAT_E_ARGUMENT;
  P.dtype = (a->flags & LEAT_FLAG_LOGITS_BF16) ? 1 : ((a->flags & LEAT_FLAG_LOGITS_F16) ? 2 : 0);
  P.out_ids = a->out_ids; P.out_greedy = a->out_greedy; P.out_cut = a->out_cut; P.out_kept = a->out_kept;
  P.out_probs = a->out_probs; P.out_prob_ids = a->out_prob_ids; P.out_width = a->out_width;
  P.status = a->status;
  P.cap = h->cap; P.keep = h->keep; P.k_max = h->k_max;
  P.ws_keys = reinterpret_cast<unsigned long long*>(h->ws + h->L.keys);
  P.ws_count = reinterpret_cast<int*>(h->ws + h->L.count);
  P.ws_best = reinterpret_cast<unsigned long long*>(h->ws + h->L.best);
  P.ws_min = reinterpret_cast<float*>(h->ws + h->L.vmin);
  P.ws_ticket = reinterpret_cast<unsigned*>(h->ws + h->L.ticket);
  P.ws_flag = reinterpret_cast<int*>(h->ws + h->L.flag);
  return LEAT_OK;
}

int pick_vec(const KParams& P) {
  const int per_vec = P.dtype == 0 ? 4 : 8;  // logits in 16 bytes
  bool ok = P.vocab % per_vec == 0 && P.row_stride % per_vec == 0 && aligned(P.logits, 16);
  if (P.seen) ok = ok && P.seen_stride % 4 == 0 && aligned(P.seen, 4);
  return ok ? 4 : 1;
}

// A launch that may begin while the kernel before it in the stream still runs (programmatic
// dependent launch); the kernel itself waits, with grid_dependency_wait(), before it reads what
// that kernel writes.
template <typename... Params, typename... Args>
cudaError_t launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t shared, cudaStream_t stream,
                             Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = shared;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, kernel, args...);
}

template <bool PEN>
int launch_one(const KParams& P, const Plan& plan, cudaStream_t stream) {
  dim3 grid(plan.slices, plan.grid_rows > 0 && plan.grid_rows < P.rows ? plan.grid_rows : P.rows);
  // after the list finish the blocks may move in early (the filter's floors and flags are final by
  // then); straight after a filter launch they must not
  const cudaError_t e = ((P.list && P.lean) || (P.shard.world > 0 && P.only_rows)) ? launch_dependent(sample_kernel<PEN>, grid, dim3(plan.threads), (size_t)plan.shared, stream, P)
                               : (sample_kernel<PEN><<<grid, plan.threads, plan.shared, stream>>>(P), cudaGetLastError());
  return cuda_failed(e, "sample_kernel launch") ? LEAT_E_CUDA : LEAT_OK;
}

int launch_sample(leat_sampler* h, KParams& P, cudaStream_t stream) {
  h->launches = 0;
  if (P.rows == 0) return LEAT_OK;
  int dev = -1;
  if (cuda_failed(cudaGetDevice(&dev), "cudaGetDevice")) return LEAT_E_CUDA;
  if (dev != h->device) return LEAT_E_DEVICE;
  if (!P.logits || (!P.out_ids && !P.cand_count && !P.out_cut)) return LEAT_E_ARGUMENT;
  const bool pen = P.seen != nullptr || P.history != nullptr;
  const int vec = pick_vec(P);
  // large aligned rows take the filter path: a floor per row, one streaming filter, then one block
  // per row finishes from the row's list
  bool filtered = h->has_list && !h->tune_no_filter && vec == 4 && !P.seen && P.vocab >= kFilterMinVocab;
  if (filtered && P.shard.world > 0) {
    // a shard with a peer exchange hands listed rows over from the list finish's block only
    int ht = 0, words = 0;
    const size_t bytes = lean_shared(P.vocab, P.history_cap, P.history != nullptr,
                                     P.history ? next_pow2(P.history_cap * 2 < 64 ? 64 : P.history_cap * 2) : 0, &ht, &words);
    if (bytes == 0 || bytes > (size_t)kMostShared) filtered = false;
  }
  // LEAT_FLAG_CLEAR_STATUS: filter_kernel clears the word on the filter path, a memset node otherwise
  if ((P.flags & LEAT_FLAG_CLEAR_STATUS) && P.status && !filtered &&
      cuda_failed(cudaMemsetAsync(P.status, 0, sizeof(int), stream), "cudaMemsetAsync")) return LEAT_E_CUDA;
  if (h->timing) {
    P.stamps = reinterpret_cast<unsigned long long*>(h->ws + h->L.stamps);
    if (cuda_failed(cudaMemsetAsync(P.stamps, 0, 16 * 8, stream), "cudaMemsetAsync")) return LEAT_E_CUDA;
  }
  // (the ring of bulk copies moves float32 logits only: 16-bit rows without a list are streamed
  // with plain loads)
  Plan plan = make_plan(h, P.rows, P.vocab, P.history_cap, P.history != nullptr, P.dtype == 0 ? vec : 1);
  P.slices = plan.slices; P.slice_len = plan.slice_len; P.bm_words = plan.bm_words; P.ht_size = plan.ht_size;
  P.ring_stages = plan.ring_stages;  // 0 unless rows are 16-byte aligned multiples of four floats
  if (plan.shared > kMostShared) return LEAT_E_CAPACITY;  // (a history this long with top_k this large)
  if (filtered) {
    P.list = reinterpret_cast<unsigned long long*>(h->ws + h->L.list);
    P.list_count = reinterpret_cast<int*>(h->ws + h->L.list_count);
    P.list_info = reinterpret_cast<unsigned long long*>(h->ws + h->L.list_info);
    P.list_cap = kListCap;
    // the rows' lists are emptied by the kernels that take them; after a failed launch, here
    if (h->dirty && (cuda_failed(cudaMemsetAsync(P.list_count, 0, (size_t)h->max_rows * 4, stream), "cudaMemsetAsync") ||
                     cuda_failed(cudaMemsetAsync(P.list_info, 0, (size_t)h->max_rows * 8, stream), "cudaMemsetAsync")))
      return LEAT_E_CUDA;
    h->dirty = 1;
    // one small block per row finishes the rows that have lists (or, for a shard with a peer
    // exchange, hands their candidates to the rows' owners); sample_kernel, after it, takes the rest
    size_t lean_bytes = 0;
    if (!P.cand_count || P.shard.world > 0) {
      lean_bytes = lean_shared(P.vocab, P.history_cap, P.history != nullptr, plan.ht_size, &P.fl_ht, &P.fl_area_words);
      if (lean_bytes > (size_t)kMostShared) lean_bytes = 0;
    }
    P.lean = lean_bytes > 0 ? 1 : 0;
    const int span = FILTER_THREADS * FILTER_VECS * (P.dtype == 0 ? 4 : 8);  // logits of one work item
    const int per_row = (P.vocab + span - 1) / span;
    const int items = per_row * P.rows;
    int blocks = items < h->sm_count * 4 ? items : h->sm_count * 4;  // four blocks fit an SM
    // few rows: every row gets blocks of its own, so that no block works out more than one floor
    int per = 0;
    if (items > blocks && h->sm_count * 4 / P.rows >= 4) {
      per = h->sm_count * 4 / P.rows;
      if (per > per_row) per = per_row;
      blocks = per * P.rows;
    }
    // Unless the rows are about as many as the blocks (then a block works out little more than one
    // floor anyway) or a mere handful, the floors are worked out first, one block per row, instead
    // of by each of the blocks that share a row (measured, us per step: 16 rows 16.8 against 19.8,
    // 72 rows 24.3 against 29.6, 256 rows 2 to 4 better, 512 rows 2 to 3 worse, a single row 13.5
    // against 12.1)
    const int floors_first = (P.rows >= 4 && P.rows * 4 < h->sm_count * 4 * 3) ? 1 : 0;
    // the first launch is a programmatic dependent of whatever comes before it in the stream (the
    // kernel that writes the logits): its blocks may be placed early, and wait before they read
    if (floors_first) {
      const cudaError_t e0 = P.dtype == 0   ? launch_dependent(floor_kernel<F32>, dim3(P.rows), dim3(SAMPLE_CHUNKS), 0, stream, P)
                             : P.dtype == 1 ? launch_dependent(floor_kernel<BF16>, dim3(P.rows), dim3(SAMPLE_CHUNKS), 0, stream, P)
                                            : launch_dependent(floor_kernel<F16>, dim3(P.rows), dim3(SAMPLE_CHUNKS), 0, stream, P);
      if (cuda_failed(e0, "floor_kernel launch")) return LEAT_E_CUDA;
      h->launches += 1;
    }
    const cudaError_t e =
        P.dtype == 0 ? launch_dependent(filter_kernel<F32>, dim3(blocks), dim3(FILTER_THREADS), kFilterAhead, stream, P, per_row, items, per, floors_first)
        : P.dtype == 1 ? launch_dependent(filter_kernel<BF16>, dim3(blocks), dim3(FILTER_THREADS), kFilterAhead, stream, P, per_row, items, per, floors_first)
                       : launch_dependent(filter_kernel<F16>, dim3(blocks), dim3(FILTER_THREADS), kFilterAhead, stream, P, per_row, items, per, floors_first);
    if (cuda_failed(e, "filter_kernel launch")) return LEAT_E_CUDA;
    h->launches += 1;
    if (P.lean) {
      // twice the threads per row while every row's block has an SM of its own (measured, us per step:
      // 72 rows 23.3 against 23.7 with 256 threads, 16 rows 16.8 against 18.1; 256 rows 66.2 against 64.9)
      const bool wide = P.rows <= h->sm_count;
      cudaError_t e2;
      if (P.shard.world > 0)
        e2 = wide ? launch_dependent(shard_select_kernel<FL_THREADS_WIDE>, dim3(P.rows), dim3(FL_THREADS_WIDE), lean_bytes, stream, P)
                  : launch_dependent(shard_select_kernel<FL_THREADS>, dim3(P.rows), dim3(FL_THREADS), lean_bytes, stream, P);
      else
        e2 = wide ? launch_dependent(finish_list_kernel<FL_THREADS_WIDE>, dim3(P.rows), dim3(FL_THREADS_WIDE), lean_bytes, stream, P)
                  : launch_dependent(finish_list_kernel<FL_THREADS>, dim3(P.rows), dim3(FL_THREADS), lean_bytes, stream, P);
      if (cuda_failed(e2, "finish_list_kernel launch")) return LEAT_E_CUDA;
      h->launches += 1;
      // ... with a short grid of blocks that look at the rows' flags and mostly leave
      const int resident = h->sm_count * 2;
      plan.grid_rows = (resident + plan.slices - 1) / plan.slices;
    }
  }
  if (P.shard.world > 0 && P.lean) {
    // the rows the select marked (no list, or a list that did not hold up) are streamed; the
    // blocks of every other row look at the marks and leave
    P.list = nullptr;
    P.lean = 0;
    P.only_rows = P.shard.marks;
  }
  int rc = pen ? launch_one<true>(P, plan, stream) : launch_one<false>(P, plan, stream);
  if (rc != LEAT_OK) return rc;
  h->launches += 1;
  if (filtered && P.cand_count && P.shard.world == 0) {
    // a shard's rows whose list did not hold up are streamed by a second launch; its blocks leave
    // at once for every other row
    P.list = nullptr;
    P.only_rows = P.cand_count;
    rc = pen ? launch_one<true>(P, plan, stream) : launch_one<false>(P, plan, stream);
    if (rc != LEAT_OK) return rc;
    h->launches += 1;
  }
  h->dirty = 0;
  return LEAT_OK;
}

template <typename K>
int allow_shared(K kernel, int bytes) {
  return cuda_failed(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes),
                     "cudaFuncSetAttribute");
}

}  // namespace

extern "C" {

size_t leat_sampler_workspace_bytes(int32_t max_rows, int32_t max_vocab, int32_t k_max) {
  if (max_rows <= 0 || max_vocab <= 0 || k_max <= 0 || k_max > kMaxK) return 0;
  return layout_for(max_rows, max_vocab, keep_for(k_max)).total;
}

int leat_sampler_create(void* workspace, size_t bytes, int32_t device, int32_t max_rows, int32_t max_vocab,
                        int32_t k_max, leat_sampler_t** out) {
  if (!workspace || !out || max_rows <= 0 || max_vocab <= 0 || k_max <= 0 || k_max > kMaxK)
    return LEAT_E_ARGUMENT;
  leat_sampler* h = new (std::nothrow) leat_sampler();
  if (!h) return LEAT_E_ARGUMENT;
  h->device = device; h->max_rows = max_rows; h->max_vocab = max_vocab; h->k_max = k_max;
  h->keep = keep_for(k_max); h->cap = cap_for(h->keep);
  h->tune_threads = 0; h->tune_slices = 0; h->tune_no_filter = 0; h->has_list = 1; h->timing = 0; h->dirty = 0; h->launches = 0;
  h->L = layout_for(max_rows, max_vocab, h->keep);
  h->ws = static_cast<unsigned char*>(workspace);
  if (bytes < h->L.total || !aligned(workspace, 256)) { delete h; return LEAT_E_WORKSPACE; }
  int dev = -1;
  if (cuda_failed(cudaGetDevice(&dev), "cudaGetDevice")) { delete h; return LEAT_E_CUDA; }
  if (dev != device) { delete h; return LEAT_E_DEVICE; }
  int sms = 0;
  if (cuda_failed(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device), "cudaDeviceGetAttribute")) {
    delete h; return LEAT_E_CUDA;
  }
  h->sm_count = sms > 0 ? sms : 148;
  const int most = kMostShared;
  if (allow_shared(sample_kernel<true>, most) || allow_shared(sample_kernel<false>, most) ||
      allow_shared(finish_candidates_kernel, most) || allow_shared(finish_list_kernel<FL_THREADS>, most) ||
      allow_shared(finish_list_kernel<FL_THREADS_WIDE>, most)) {
    delete h; return LEAT_E_CUDA;
  }
  if (cuda_failed(cudaMemset(workspace, 0, h->L.total), "cudaMemset") ||
      cuda_failed(cudaDeviceSynchronize(), "cudaDeviceSynchronize")) {
    delete h; return LEAT_E_CUDA;
  }
  *out = h;
  return LEAT_OK;
}

int leat_sampler_destroy(leat_sampler_t* handle) {
  delete handle;
  return LEAT_OK;
}

int leat_sampler_tune(leat_sampler_t* h, int32_t threads, int32_t slices) {
  if (!h) return LEAT_E_ARGUMENT;
  if (threads != 0 && threads != 128 && threads != 256 && threads != 512) return LEAT_E_ARGUMENT;
  if (slices < 0) return LEAT_E_ARGUMENT;
  h->tune_threads = threads; h->tune_slices = slices;
  return LEAT_OK;
}

int leat_sampler_tune_filter(leat_sampler_t* h, int32_t enabled) {
  if (!h) return LEAT_E_ARGUMENT;
  h->tune_no_filter = enabled ? 0 : 1;
  return LEAT_OK;
}

int leat_sampler_plan(const leat_sampler_t* h, int32_t rows, int32_t vocab, int32_t history_cap,
                      int32_t* threads, int32_t* slices, int32_t* shared) {
  if (!h || rows <= 0 || vocab <= 0) return LEAT_E_ARGUMENT;
  Plan p = make_plan(h, rows, vocab, history_cap, history_cap > 0, vocab % 4 == 0 ? 4 : 1);
  if (threads) *threads = p.threads;
  if (slices) *slices = p.slices;
  if (shared) *shared = p.shared;
  return LEAT_OK;
}

int leat_sampler_last_launches(const leat_sampler_t* h) { return h ? h->launches : 0; }

int leat_sampler_time_kernels(leat_sampler_t* h, int32_t enabled) {
  if (!h) return LEAT_E_ARGUMENT;
  h->timing = enabled ? 1 : 0;
  return LEAT_OK;
}

int leat_sampler_kernel_times(leat_sampler_t* h, float* milliseconds) {
  if (!h || !milliseconds || !h->timing) return LEAT_E_ARGUMENT;
  unsigned long long stamps[16];
  if (cuda_failed(cudaDeviceSynchronize(), "cudaDeviceSynchronize") ||
      cuda_failed(cudaMemcpy(stamps, h->ws + h->L.stamps, sizeof(stamps), cudaMemcpyDeviceToHost), "cudaMemcpy"))
    return LEAT_E_CUDA;
  unsigned long long first = ~0ull;
  for (int k = 0; k < 6; ++k)
    if (stamps[2 * k] && ~stamps[2 * k] < first) first = ~stamps[2 * k];
  for (int k = 0; k < 6; ++k) {
    const bool ran = stamps[2 * k] != 0ull;
    milliseconds[2 * k] = ran ? (float)((double)(~stamps[2 * k] - first) * 1e-6) : -1.0f;
    milliseconds[2 * k + 1] = ran ? (float)((double)(stamps[2 * k + 1] - first) * 1e-6) : -1.0f;
  }
  return LEAT_OK;
}

const char* leat_sampler_last_cuda_error(void) { return g_cuda_error; }

int leat_sample(leat_sampler_t* h, const leat_sample_args* a, leat_stream_t stream) {
  KParams P;
  int rc = fill_params(h, a, P);
  if (rc != LEAT_OK) return rc;
  if (a->rows == 0) {
    h->launches = 0;
    if ((a->flags & LEAT_FLAG_CLEAR_STATUS) && a->status &&
        cuda_failed(cudaMemsetAsync(a->status, 0, sizeof(int), static_cast<cudaStream_t>(stream)), "cudaMemsetAsync"))
      return LEAT_E_CUDA;
    return LEAT_OK;
  }
  if (!a->out_ids) return LEAT_E_ARGUMENT;
  return launch_sample(h, P, static_cast<cudaStream_t>(stream));
}

int leat_argmax(leat_sampler_t* h, const float* x, int32_t rows, int32_t vocab, int64_t row_stride,
                int32_t* out, int32_t* status, leat_stream_t stream) {
  leat_sample_args a;
  memset(&a, 0, sizeof(a));
  a.logits = x; a.rows = rows; a.vocab = vocab; a.row_stride = row_stride;
  a.out_ids = out; a.status = status;
  KParams P;
  int rc = fill_params(h, &a, P);
  if (rc != LEAT_OK) return rc;
  if (!out) return LEAT_E_ARGUMENT;
  P.force_greedy = 1;
  if (pick_vec(P) == 4 && vocab >= kArgmaxMinVocab && rows <= 65535 && !h->tune_no_filter) {
    // rows of whole aligned vectors: one launch of a kernel of its own
    h->launches = 0;
    if (rows == 0) return LEAT_OK;
    int dev = -1;
    if (cuda_failed(cudaGetDevice(&dev), "cudaGetDevice")) return LEAT_E_CUDA;
    if (dev != h->device) return LEAT_E_DEVICE;
    // enough blocks to fill the GPU, none with less than one round of loads to do, and with many
    // rows two rounds a block: short blocks, handed out as SMs fall free, leave no tail (measured,
    // 256 x 262144: 40.5 us against 45.7 with a third of a row per block)
    int slices = (h->sm_count * 4 + rows - 1) / rows;
    const int rounds = (vocab + AM_ROUND - 1) / AM_ROUND;
    if (slices < (rounds + 1) / 2) slices = (rounds + 1) / 2;
    if (slices > rounds) slices = rounds;
    if (slices > AM_MAX_SLICES) slices = AM_MAX_SLICES;
    if (slices < 1) slices = 1;
    const int span = round_up((vocab + slices - 1) / slices, 1024);
    slices = (vocab + span - 1) / span;
    const cudaError_t e = launch_dependent(argmax_kernel, dim3(slices, rows), dim3(AM_THREADS), 0, static_cast<cudaStream_t>(stream),
                                           x, (int)vocab, (long long)row_stride, slices, span,
                                           reinterpret_cast<unsigned long long*>(h->ws + h->L.keys),
                                           reinterpret_cast<unsigned*>(h->ws + h->L.ticket), (int*)out);
    if (cuda_failed(e, "argmax_kernel launch")) return LEAT_E_CUDA;
    h->launches = 1;
    return LEAT_OK;
  }
  return launch_sample(h, P, static_cast<cudaStream_t>(stream));
}

int leat_cutoff(leat_sampler_t* h, const float* scores, int32_t rows, int32_t vocab, int64_t row_stride,
                const float* top_k, const float* top_p, const float* min_p, float* cut, int32_t* status,
                leat_stream_t stream) {
  if (!top_k || !top_p || !min_p || !cut) return LEAT_E_ARGUMENT;
  leat_sample_args a;
  memset(&a, 0, sizeof(a));
  a.logits = scores; a.rows = rows; a.vocab = vocab; a.row_stride = row_stride;
  a.out_cut = cut; a.status = status;
  KParams P;
  int rc = fill_params(h, &a, P);
  if (rc != LEAT_OK) return rc;
  P.opt_k = top_k; P.opt_p = top_p; P.opt_m = min_p;
  return launch_sample(h, P, static_cast<cudaStream_t>(stream));
}

int leat_verify_draft(const int32_t* drafted, const int32_t* sampled, const int32_t* greedy, int32_t n,
                      int32_t drafts, int32_t* accepted, int32_t* tokens, leat_stream_t stream) {
  if (!sampled || !accepted || !tokens || n < 0 || drafts < 0 || (drafts > 0 && !drafted)) return LEAT_E_ARGUMENT;
  if (n == 0) return LEAT_OK;
  verify_kernel<<<(n + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(drafted, sampled, greedy, n,
                                                                                drafts, accepted, tokens);
  return cuda_failed(cudaGetLastError(), "verify_kernel launch") ? LEAT_E_CUDA : LEAT_OK;
}

int leat_settle_draft(const int32_t* accepted, const int32_t* last, const int32_t* drafted, const int32_t* sampled,
                      const int32_t* slots, int32_t n, int32_t drafts, int32_t* history_ids, int32_t* history_count,
                      int32_t capacity, const uint8_t* text, int32_t vocab, int32_t* next, int32_t* row,
                      leat_stream_t stream) {
  if (!accepted || !last || !sampled || !history_ids || !history_count || n < 0 || drafts < 0 || capacity <= 0 ||
      vocab <= 0 || (drafts > 0 && !drafted))
    return LEAT_E_ARGUMENT;
  if (n == 0) return LEAT_OK;
  settle_kernel<<<(n + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      accepted, last, drafted, sampled, slots, n, drafts, history_ids, history_count, capacity, text, vocab, next, row);
  return cuda_failed(cudaGetLastError(), "settle_kernel launch") ? LEAT_E_CUDA : LEAT_OK;
}

int leat_topk_local(leat_sampler_t* h, const leat_sample_args* a, float* cand_value, int32_t* cand_id,
                    int32_t* cand_count, uint64_t* best, int32_t cap, leat_stream_t stream) {
  if (!cand_value || !cand_id || !cand_count || !best || cap <= 0) return LEAT_E_ARGUMENT;
  KParams P;
  int rc = fill_params(h, a, P);
  if (rc != LEAT_OK) return rc;
  if (a->softcap > 0.0f) return LEAT_E_ARGUMENT;  // (a soft cap goes with the list finish: use leat_shard_select)
  P.cand_value = cand_value; P.cand_id = cand_id; P.cand_count = cand_count;
  P.cand_best = reinterpret_cast<unsigned long long*>(best); P.cand_cap = cap;
  return launch_sample(h, P, static_cast<cudaStream_t>(stream));
}

namespace {
int finish_from(leat_sampler* h, const leat_sample_args* a, const float* cand_value, const int32_t* cand_id,
                const int32_t* cand_count, const uint64_t* best, long long stride_value, long long stride_id,
                long long stride_count, long long stride_best, int32_t parts, int32_t cap, cudaStream_t stream) {
  if (!cand_value || !cand_id || !cand_count || !best || cap <= 0 || parts <= 0) return LEAT_E_ARGUMENT;
  if (!h || !a) return LEAT_E_ARGUMENT;
  // the handle is sized for this rank's slice; here `vocab` is the whole vocabulary's size
  leat_sample_args whole = *a;
  const int vocab = a->vocab_total > 0 ? a->vocab_total : a->vocab;
  whole.vocab = 1;
  whole.vocab_total = 0;
  KParams P;
  int rc = fill_params(h, &whole, P);
  if (rc != LEAT_OK) return rc;
  if (!a->out_ids || vocab <= 0) return LEAT_E_ARGUMENT;
  P.vocab = vocab; P.vocab_total = vocab;
  h->launches = 0;
  if (P.rows == 0) return LEAT_OK;
  int dev = -1;
  if (cuda_failed(cudaGetDevice(&dev), "cudaGetDevice")) return LEAT_E_CUDA;
  if (dev != h->device) return LEAT_E_DEVICE;
  P.g_value = cand_value; P.g_id = cand_id; P.g_count = cand_count;
  P.g_best = reinterpret_cast<const unsigned long long*>(best); P.g_parts = parts; P.cand_cap = cap;
  P.g_stride_value = stride_value; P.g_stride_id = stride_id; P.g_stride_count = stride_count; P.g_stride_best = stride_best;
  if ((P.flags & LEAT_FLAG_CLEAR_STATUS) && P.status &&
      cuda_failed(cudaMemsetAsync(P.status, 0, sizeof(int), stream), "cudaMemsetAsync")) return LEAT_E_CUDA;
  const int threads = 512;
  const int shared = (int)shared_bytes(h->cap, h->keep, 0);
  finish_candidates_kernel<<<P.rows, threads, shared, stream>>>(P);
  if (cuda_failed(cudaGetLastError(), "finish_candidates_kernel launch")) return LEAT_E_CUDA;
  h->launches = 1;
  return LEAT_OK;
}

size_t record_offsets(int rows, int cap, size_t* id_at, size_t* count_at, size_t* best_at) {
  const size_t values = (size_t)rows * cap * 4;
  *id_at = values;
  *count_at = 2 * values;
  *best_at = (2 * values + (size_t)rows * 4 + 7) / 8 * 8;
  return (*best_at + (size_t)rows * 8 + 255) / 256 * 256;
}
}  // namespace

int leat_sample_from_candidates(leat_sampler_t* h, const leat_sample_args* a, const float* cand_value,
                                const int32_t* cand_id, const int32_t* cand_count, const uint64_t* best,
                                int32_t parts, int32_t cap, leat_stream_t stream) {
  if (!a) return LEAT_E_ARGUMENT;
  const long long rows = a->rows;
  return finish_from(h, a, cand_value, cand_id, cand_count, best, rows * cap, rows * cap, rows, rows, parts, cap,
                     static_cast<cudaStream_t>(stream));
}

size_t leat_candidate_record_bytes(int32_t rows, int32_t cap) {
  if (rows <= 0 || cap <= 0) return 0;
  size_t i, c, b;
  return record_offsets(rows, cap, &i, &c, &b);
}

int leat_candidate_record_layout(int32_t rows, int32_t cap, size_t* id_at, size_t* count_at, size_t* best_at) {
  if (rows <= 0 || cap <= 0 || !id_at || !count_at || !best_at) return LEAT_E_ARGUMENT;
  record_offsets(rows, cap, id_at, count_at, best_at);
  return LEAT_OK;
}

int leat_sample_from_records(leat_sampler_t* h, const leat_sample_args* a, const void* records, int32_t parts,
                             int32_t cap, leat_stream_t stream) {
  if (!a || !records) return LEAT_E_ARGUMENT;
  size_t id_at, count_at, best_at;
  const size_t bytes = record_offsets(a->rows > 0 ? a->rows : 1, cap > 0 ? cap : 1, &id_at, &count_at, &best_at);
  const unsigned char* base = static_cast<const unsigned char*>(records);
  return finish_from(h, a, reinterpret_cast<const float*>(base), reinterpret_cast<const int32_t*>(base + id_at),
                     reinterpret_cast<const int32_t*>(base + count_at), reinterpret_cast<const uint64_t*>(base + best_at),
                     (long long)(bytes / 4), (long long)(bytes / 4), (long long)(bytes / 4), (long long)(bytes / 8),
                     parts, cap, static_cast<cudaStream_t>(stream));
}

// ---- sampling without any allocation -------------------------------------------------------------
//
// Some callers cannot hand the library a workspace because they cannot allocate device memory at
// the point of the call at all: an inference server that has already given every free byte to its
// KV-cache pool, a host binding (cgo, JNI, ctypes) that only ever receives device pointers from its
// framework and has no allocator of its own, or a step running where cudaMalloc's implicit
// device-wide synchronisation is not acceptable.  For them leat_sample_static() keeps the scratch
// the slices of a row exchange in a fixed array inside the library's own device image.
constexpr int kStaticRows = 64;
constexpr int kStaticVocab = 1 << 18;
constexpr int kStaticK = 64;
constexpr int kStaticCells = 1024;  // blocks of one call: rows x slices

constexpr size_t static_region(size_t bytes) { return (bytes + 255) / 256 * 256; }
constexpr int kStaticKeep = (kStaticK + 64 + 63) / 64 * 64;
constexpr size_t kStaticBytes = static_region((size_t)kStaticCells * kStaticKeep * 8) +
                                static_region((size_t)kStaticCells * 4) + static_region((size_t)kStaticCells * 16) +
                                static_region((size_t)kStaticCells * 4) + 2 * static_region((size_t)kStaticRows * 4);

// Every GPU that loads the library holds this array (about 1.1 MB) until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

namespace {

struct StaticDevice {
  bool ready;
  leat_sampler handle;
};
StaticDevice g_static_devices[64];
std::mutex g_static_lock;  // the first call on a device sets its entry up; threads may race to it

// Once per device, with that device current: the array's name is only a host-side stand-in, so
// ask the runtime for the device address kernels can use.
int static_setup(int device, StaticDevice** out) {
  if (device < 0 || device >= 64) return LEAT_E_DEVICE;
  StaticDevice& sd = g_static_devices[device];
  std::lock_guard<std::mutex> guard(g_static_lock);
  if (!sd.ready) {
    void* scratch = nullptr;
    if (cuda_failed(cudaGetSymbolAddress(&scratch, g_static_scratch), "cudaGetSymbolAddress")) return LEAT_E_CUDA;
    leat_sampler& h = sd.handle;
    h.device = device; h.max_rows = kStaticRows; h.max_vocab = kStaticVocab; h.k_max = kStaticK;
    h.keep = keep_for(kStaticK); h.cap = cap_for(h.keep);
    h.tune_threads = 0; h.tune_slices = 0; h.tune_no_filter = 0; h.has_list = 0; h.timing = 0; h.dirty = 0; h.launches = 0;
    Layout& L = h.L;
    L.cells = kStaticCells;
    size_t at = 0;
    auto take = [&](size_t bytes) { size_t here = at; at += static_region(bytes); return here; };
    L.keys = take((size_t)L.cells * h.keep * 8);
    L.count = take((size_t)L.cells * 4);
    L.best = take((size_t)L.cells * 16);
    L.vmin = take((size_t)L.cells * 4);
    L.ticket = take((size_t)kStaticRows * 4);
    L.flag = take((size_t)kStaticRows * 4);
    L.list = 0; L.list_count = 0; L.list_info = 0; L.stamps = 0;  // the fixed scratch has no room for lists: the fused path is used
    L.total = at;
    if (L.total > kStaticBytes || h.keep != kStaticKeep) return LEAT_E_WORKSPACE;
    h.ws = static_cast<unsigned char*>(scratch);
    int sms = 0;
    if (cuda_failed(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device), "cudaDeviceGetAttribute"))
      return LEAT_E_CUDA;
    h.sm_count = sms > 0 ? sms : 148;
    const int most = kMostShared;
    if (allow_shared(sample_kernel<true>, most) || allow_shared(sample_kernel<false>, most))
      return LEAT_E_CUDA;
    sd.ready = true;
  }
  *out = &sd;
  return LEAT_OK;
}

}  // namespace

int leat_sample_static(const leat_sample_args* a, leat_stream_t stream) {
  if (!a || !a->out_ids) return LEAT_E_ARGUMENT;
  if (a->rows > kStaticRows || a->vocab > kStaticVocab) return LEAT_E_CAPACITY;
  if (a->flags & (LEAT_FLAG_LOGITS_BF16 | LEAT_FLAG_LOGITS_F16)) return LEAT_E_ARGUMENT;  // float32 logits only
  if (a->rows == 0) {  // nothing to sample; the status word is still cleared on request, as leat_sample does
    if (a->vocab <= 0) return LEAT_E_ARGUMENT;
    if ((a->flags & LEAT_FLAG_CLEAR_STATUS) && a->status &&
        cuda_failed(cudaMemsetAsync(a->status, 0, sizeof(int), static_cast<cudaStream_t>(stream)), "cudaMemsetAsync"))
      return LEAT_E_CUDA;
    return LEAT_OK;
  }
  int device = -1;
  if (cuda_failed(cudaGetDevice(&device), "cudaGetDevice")) return LEAT_E_CUDA;
  StaticDevice* sd = nullptr;
  int rc = static_setup(device, &sd);
  if (rc != LEAT_OK) return rc;
  leat_sampler* h = &sd->handle;
  KParams P;
  rc = fill_params(h, a, P);
  if (rc != LEAT_OK) return rc;
  // the array keeps what the last call left: the words that count a row's finished slices and mark
  // rows for the multi-pass kernel must start at zero
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cuda_failed(cudaMemsetAsync(h->ws + h->L.ticket, 0, h->L.total - h->L.ticket, s), "cudaMemsetAsync"))
    return LEAT_E_CUDA;
  return launch_sample(h, P, s);
}

// ---- vocabulary shards with a peer exchange ------------------------------------------------------

struct leat_shard {
  leat_sampler* h;
  ShardView view;
  int finish_shared;
};

namespace {
// the rank's own words behind the exchange part of its region: step number, tickets, marks
size_t shard_private_at(int world, int owned, int cap) { return shard_region_bytes(world, owned, cap); }
size_t shard_private_bytes(int rows) { return 256 + ((size_t)rows * 4 + 255) / 256 * 256; }
}  // namespace

size_t leat_shard_region_bytes(int32_t rows, int32_t cap, int32_t world) {
  if (rows <= 0 || cap <= 0 || world <= 0 || world > SHARD_MAX_WORLD) return 0;
  const int owned = (rows + world - 1) / world;
  return shard_private_at(world, owned, cap) + shard_private_bytes(rows);
}

int leat_peer_alloc(size_t bytes, void** ptr, unsigned char* handle) {
  if (!ptr || !handle || bytes == 0) return LEAT_E_ARGUMENT;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is exchanged as 64 bytes");
  void* p = nullptr;
  if (cuda_failed(cudaMalloc(&p, bytes), "cudaMalloc")) return LEAT_E_CUDA;
  cudaIpcMemHandle_t ipc;
  if (cuda_failed(cudaMemset(p, 0, bytes), "cudaMemset") || cuda_failed(cudaDeviceSynchronize(), "cudaDeviceSynchronize") ||
      cuda_failed(cudaIpcGetMemHandle(&ipc, p), "cudaIpcGetMemHandle")) {
    cudaFree(p);
    return LEAT_E_CUDA;
  }
  memcpy(handle, &ipc, 64);
  *ptr = p;
  return LEAT_OK;
}

int leat_peer_open(const unsigned char* handle, void** ptr) {
  if (!ptr || !handle) return LEAT_E_ARGUMENT;
  cudaIpcMemHandle_t ipc;
  memcpy(&ipc, handle, 64);
  return cuda_failed(cudaIpcOpenMemHandle(ptr, ipc, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle") ? LEAT_E_CUDA : LEAT_OK;
}

int leat_peer_close(void* ptr) {
  return cuda_failed(cudaIpcCloseMemHandle(ptr), "cudaIpcCloseMemHandle") ? LEAT_E_CUDA : LEAT_OK;
}

int leat_peer_free(void* ptr) { return cuda_failed(cudaFree(ptr), "cudaFree") ? LEAT_E_CUDA : LEAT_OK; }

int leat_shard_create(leat_sampler_t* h, int32_t rank, int32_t world, int32_t rows, int32_t cap, void* const* regions,
                      leat_shard_t** out) {
  if (!h || !regions || !out || world <= 0 || world > SHARD_MAX_WORLD || rank < 0 || rank >= world || rows <= 0 || cap <= 0)
    return LEAT_E_ARGUMENT;
  if (rows > h->max_rows || cap > FL_SORT) return LEAT_E_CAPACITY;
  leat_shard* s = new (std::nothrow) leat_shard();
  if (!s) return LEAT_E_ARGUMENT;
  s->h = h;
  ShardView& v = s->view;
  memset(&v, 0, sizeof(v));
  for (int r = 0; r < world; ++r) {
    if (!regions[r]) { delete s; return LEAT_E_ARGUMENT; }
    v.region[r] = static_cast<unsigned char*>(regions[r]);
  }
  v.rank = rank; v.world = world; v.rows = rows; v.owned = (rows + world - 1) / world; v.cap = cap;
  unsigned char* mine = v.region[rank] + shard_private_at(world, v.owned, cap);
  v.epoch = reinterpret_cast<unsigned*>(mine);
  v.tickets = v.epoch + 8;
  v.done_ticket = v.epoch + 24;
  v.marks = reinterpret_cast<int*>(mine + 256);
  const unsigned one = 1u;  // steps count from 1: a region is all zeros before its first step
  if (cuda_failed(cudaMemcpy(v.epoch, &one, sizeof(one), cudaMemcpyHostToDevice), "cudaMemcpy")) { delete s; return LEAT_E_CUDA; }
  s->finish_shared = FL_FIXED + FL_HIST_WORDS * 4 + FL_KEYS * 8 + FL_AREA_MIN_WORDS * 4;
  const int most = kMostShared;
  if (allow_shared(shard_select_kernel<FL_THREADS>, most) || allow_shared(shard_select_kernel<FL_THREADS_WIDE>, most) ||
      allow_shared(shard_finish_kernel<FL_THREADS>, most) || allow_shared(shard_finish_kernel<FL_THREADS_WIDE>, most)) {
    delete s;
    return LEAT_E_CUDA;
  }
  *out = s;
  return LEAT_OK;
}

int leat_shard_destroy(leat_shard_t* shard) {
  delete shard;
  return LEAT_OK;
}

int leat_shard_select(leat_shard_t* s, const leat_sample_args* a, leat_stream_t stream) {
  if (!s || !a) return LEAT_E_ARGUMENT;
  if (a->rows != s->view.rows) return LEAT_E_ARGUMENT;
  KParams P;
  int rc = fill_params(s->h, a, P);
  if (rc != LEAT_OK) return rc;
  P.shard = s->view;
  P.cand_count = s->view.marks;  // (what marks the call as a shard's for the streaming kernel)
  P.cand_cap = s->view.cap;
  return launch_sample(s->h, P, static_cast<cudaStream_t>(stream));
}

namespace {
int shard_tail(leat_shard* s, const leat_sample_args* a, KParams& P) {
  if (!s || !a) return LEAT_E_ARGUMENT;
  if (a->rows != s->view.rows) return LEAT_E_ARGUMENT;
  // the handle is sized for this rank's slice; here `vocab` is the whole vocabulary's size
  leat_sample_args whole = *a;
  const int vocab = a->vocab_total > 0 ? a->vocab_total : a->vocab;
  whole.vocab = 1;
  whole.vocab_total = 0;
  int rc = fill_params(s->h, &whole, P);
  if (rc != LEAT_OK) return rc;
  if (!a->out_ids || vocab <= 0) return LEAT_E_ARGUMENT;
  P.vocab = vocab; P.vocab_total = vocab;
  P.shard = s->view;
  if (s->h->timing) P.stamps = reinterpret_cast<unsigned long long*>(s->h->ws + s->h->L.stamps);
  int dev = -1;
  if (cuda_failed(cudaGetDevice(&dev), "cudaGetDevice")) return LEAT_E_CUDA;
  if (dev != s->h->device) return LEAT_E_DEVICE;
  return LEAT_OK;
}
}  // namespace

int leat_shard_finish(leat_shard_t* s, const leat_sample_args* a, leat_stream_t stream) {
  KParams P;
  int rc = shard_tail(s, a, P);
  if (rc != LEAT_OK) return rc;
  const ShardView& v = s->view;
  const int mine = v.rows - v.rank * v.owned < v.owned ? v.rows - v.rank * v.owned : v.owned;
  s->h->launches = 0;
  if (mine <= 0) return LEAT_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool wide = mine <= s->h->sm_count;  // (as for the list finish: a block of 512 threads while each has an SM of its own)
  const cudaError_t e =
      wide ? launch_dependent(shard_finish_kernel<FL_THREADS_WIDE>, dim3(mine), dim3(FL_THREADS_WIDE), (size_t)s->finish_shared, st, P)
           : launch_dependent(shard_finish_kernel<FL_THREADS>, dim3(mine), dim3(FL_THREADS), (size_t)s->finish_shared, st, P);
  if (cuda_failed(e, "shard_finish_kernel launch")) return LEAT_E_CUDA;
  s->h->launches = 1;
  return LEAT_OK;
}

int leat_shard_result(leat_shard_t* s, const leat_sample_args* a, leat_stream_t stream) {
  KParams P;
  int rc = shard_tail(s, a, P);
  if (rc != LEAT_OK) return rc;
  if (cuda_failed(launch_dependent(shard_result_kernel, dim3(1), dim3(256), 0, static_cast<cudaStream_t>(stream), P),
                  "shard_result_kernel launch")) return LEAT_E_CUDA;
  s->h->launches = 1;
  return LEAT_OK;
}

}  // extern "C"

// Host-side continuous-batching scheduler and paged-KV block allocator.
//
// The scheduler owns three pieces of state: a free list of KV pages, a table of decode slots
// (one per running sequence, lowest free index first so the active prefix stays dense), and a
// FIFO of waiting requests.  It never looks at device memory: sequence lengths advance
// deterministically by one token per decode step, so page demand is known on the host; the
// engine tells it when a slot finished.  Admission respects the slot limit, the page budget
// (all pages of the prompt are reserved at admission, also when the prompt is prefilled in several
// chunks; decode pages on demand) and a per-step prefill token budget; prompts
// longer than the budget are prefilled in chunks.
//
// Behaviourally this is the role of InferenceBatchState in the reference
// (areno/engine/data/rollout_state.py:20-242), restated as a C++ component behind a C ABI.
#include <algorithm>
#include <cstdint>
#include <deque>
#include <vector>

namespace {

struct Request {
  long long id;
  int prompt_len;
  int max_new;
};

struct Slot {
  bool used = false;
  bool prefilling = false;
  long long req_id = -1;
  int prompt_len = 0;
  int prefilled = 0;    // prompt tokens already run through the model
  int seq_len = 0;      // tokens with KV in the cache (after the current step is planned)
  int max_len = 0;      // prompt_len + max_new
  long long admit_order = 0;  // position in the admission sequence (larger = admitted later)
  std::vector<int> pages;
};

struct Scheduler {
  int max_slots, num_pages, page_size, max_pages_per_seq, max_prefill_tokens;
  std::vector<int> free_pages;
  std::vector<Slot> slots;
  std::deque<Request> waiting;
  int running = 0;
  long long admitted_total = 0;

  Scheduler(int ms, int np, int ps, int mpps, int mpt)
      : max_slots(ms), num_pages(np), page_size(ps), max_pages_per_seq(mpps), max_prefill_tokens(mpt), slots(ms) {
    free_pages.reserve(np);
    for (int p = np - 1; p >= 0; --p) free_pages.push_back(p);
  }

  int pages_for(int tokens) const { return (tokens + page_size - 1) / page_size; }

  bool grow(Slot& s, int tokens) {
    const int need = pages_for(tokens);
    if (need > max_pages_per_seq) return false;
    const int extra = need - static_cast<int>(s.pages.size());
    if (extra <= 0) return true;
    if (extra > static_cast<int>(free_pages.size())) return false;
    for (int i = 0; i < extra; ++i) {
      s.pages.push_back(free_pages.back());
      free_pages.pop_back();
    }
    return true;
  }

  void release(Slot& s) {
    for (int p : s.pages) free_pages.push_back(p);
    s.pages.clear();
    s.used = false;
    s.prefilling = false;
    s.req_id = -1;
  }
};

}  // namespace

extern "C" {

void* areno_sched_create(int max_slots, int num_pages, int page_size, int max_pages_per_seq, int max_prefill_tokens) {
  if (max_slots <= 0 || num_pages <= 0 || page_size <= 0) return nullptr;
  return new Scheduler(max_slots, num_pages, page_size, max_pages_per_seq, max_prefill_tokens);
}

void areno_sched_destroy(void* h) { delete static_cast<Scheduler*>(h); }

int areno_sched_add(void* h, long long req_id, int prompt_len, int max_new) {
  auto* s = static_cast<Scheduler*>(h);
  if (prompt_len <= 0) return -1;
  if (s->pages_for(prompt_len + std::max(max_new, 0)) > s->max_pages_per_seq) return -2;
  s->waiting.push_back(Request{req_id, prompt_len, max_new});
  return 0;
}

// Plan one prefill step.  First continues slots that are mid-prompt, then admits waiting
// requests in FIFO order while slots, pages and the token budget allow.  Each output entry is a
// (slot, request, first prompt token, token count, last-chunk flag).  Returns the entry count.
int areno_sched_plan_prefill(void* h, int max_out, int* out_slot, long long* out_req, int* out_start, int* out_len,
                             int* out_last) {
  auto* s = static_cast<Scheduler*>(h);
  int budget = s->max_prefill_tokens;
  int n = 0;
  auto emit = [&](int slot_idx) {
    Slot& sl = s->slots[slot_idx];
    const int remaining = sl.prompt_len - sl.prefilled;
    const int take = std::min(remaining, budget);
    if (take <= 0 || n >= max_out) return false;
    if (!s->grow(sl, sl.prefilled + take + 1)) return false;  // +1: room for the first decoded token
    out_slot[n] = slot_idx;
    out_req[n] = sl.req_id;
    out_start[n] = sl.prefilled;
    out_len[n] = take;
    sl.prefilled += take;
    sl.seq_len = sl.prefilled;
    const bool last = sl.prefilled == sl.prompt_len;
    out_last[n] = last ? 1 : 0;
    if (last) sl.prefilling = false;
    budget -= take;
    ++n;
    return true;
  };
  for (int i = 0; i < s->max_slots && budget > 0; ++i)
    if (s->slots[i].used && s->slots[i].prefilling) emit(i);
  while (!s->waiting.empty() && budget > 0 && n < max_out) {
    int free_slot = -1;
    for (int i = 0; i < s->max_slots; ++i)
      if (!s->slots[i].used) { free_slot = i; break; }
    if (free_slot < 0) break;
    const Request r = s->waiting.front();
    // Admit only if the whole prompt (plus one decode token) fits in free pages right now, and take
    // those pages immediately: a prompt that is prefilled over several steps keeps its claim, so a
    // later admission or a growing decoder cannot leave it stranded half-way.
    if (s->pages_for(r.prompt_len + 1) > static_cast<int>(s->free_pages.size())) break;
    Slot& sl = s->slots[free_slot];
    sl.used = true;
    sl.prefilling = true;
    sl.req_id = r.id;
    sl.prompt_len = r.prompt_len;
    sl.prefilled = 0;
    sl.seq_len = 0;
    sl.max_len = r.prompt_len + r.max_new;
    sl.admit_order = s->admitted_total;
    if (!s->grow(sl, r.prompt_len + 1) || !emit(free_slot)) {
      s->release(sl);
      break;
    }
    s->waiting.pop_front();
    ++s->running;
    ++s->admitted_total;
  }
  return n;
}

// Reserve KV room for `steps` more decoded tokens on every slot that is decoding (not mid-prompt).
// New (slot, page index, page id) triples are written to the update arrays.  Returns the number of
// updates.  The call either serves every slot or changes nothing: when the free pages do not cover
// the demand it returns -(slot+1) of the first slot (in index order) whose share would not fit, and
// when the update arrays are too short it returns -(max_slots+1); in both cases no page has moved, so
// the caller can make room (preempt a sequence) and call again without losing an update.
int areno_sched_reserve_decode(void* h, int steps, int max_upd, int* upd_slot, int* upd_index, int* upd_page) {
  auto* s = static_cast<Scheduler*>(h);
  long long need_total = 0;
  const long long have = static_cast<long long>(s->free_pages.size());
  for (int i = 0; i < s->max_slots; ++i) {
    const Slot& sl = s->slots[i];
    if (!sl.used || sl.prefilling) continue;
    const int target = std::min(sl.seq_len + steps, sl.max_len);
    const int need = s->pages_for(target);
    if (need > s->max_pages_per_seq) return -(i + 1);
    const int extra = need - static_cast<int>(sl.pages.size());
    if (extra <= 0) continue;
    need_total += extra;
    if (need_total > have) return -(i + 1);
  }
  if (need_total > max_upd) return -(s->max_slots + 1);
  int n = 0;
  for (int i = 0; i < s->max_slots; ++i) {
    Slot& sl = s->slots[i];
    if (!sl.used || sl.prefilling) continue;
    const int target = std::min(sl.seq_len + steps, sl.max_len);
    const size_t before = sl.pages.size();
    s->grow(sl, target);  // cannot fail: the demand was checked above
    for (size_t k = before; k < sl.pages.size(); ++k) {
      upd_slot[n] = i;
      upd_index[n] = static_cast<int>(k);
      upd_page[n] = sl.pages[k];
      ++n;
    }
  }
  return n;
}

// The decoding slot that was admitted last (the cheapest one to send back to the queue), or -1 when
// fewer than two sequences are decoding (evicting the only one would make no room for anybody).
int areno_sched_preempt_victim(void* h) {
  auto* s = static_cast<Scheduler*>(h);
  int victim = -1, decoding = 0;
  for (int i = 0; i < s->max_slots; ++i) {
    const Slot& sl = s->slots[i];
    if (!sl.used || sl.prefilling) continue;
    ++decoding;
    if (victim < 0 || sl.admit_order > s->slots[victim].admit_order) victim = i;
  }
  return decoding >= 2 ? victim : -1;
}

// Send the sequence in `slot` back to the head of the waiting queue: its pages are freed and it will
// be admitted again as a request with `prompt_len` prompt tokens (the original prompt plus whatever
// it had generated) and `max_new` tokens still to produce.
int areno_sched_requeue(void* h, int slot, int prompt_len, int max_new) {
  auto* s = static_cast<Scheduler*>(h);
  if (slot < 0 || slot >= s->max_slots || !s->slots[slot].used || prompt_len <= 0) return -1;
  const long long id = s->slots[slot].req_id;
  s->release(s->slots[slot]);
  --s->running;
  s->waiting.push_front(Request{id, prompt_len, std::max(max_new, 0)});
  return 0;
}

// Account for `steps` decode steps having been launched (every decoding slot grew by that much,
// capped at its maximum length).
void areno_sched_advance(void* h, int steps) {
  auto* s = static_cast<Scheduler*>(h);
  for (auto& sl : s->slots)
    if (sl.used && !sl.prefilling) sl.seq_len = std::min(sl.seq_len + steps, sl.max_len);
}

int areno_sched_finish(void* h, int slot) {
  auto* s = static_cast<Scheduler*>(h);
  if (slot < 0 || slot >= s->max_slots || !s->slots[slot].used) return -1;
  s->release(s->slots[slot]);
  --s->running;
  return 0;
}

int areno_sched_slot_pages(void* h, int slot, int* out, int max_out) {
  auto* s = static_cast<Scheduler*>(h);
  if (slot < 0 || slot >= s->max_slots) return -1;
  const auto& p = s->slots[slot].pages;
  const int n = std::min<int>(static_cast<int>(p.size()), max_out);
  for (int i = 0; i < n; ++i) out[i] = p[i];
  return static_cast<int>(p.size());
}

int areno_sched_slot_seq_len(void* h, int slot) {
  auto* s = static_cast<Scheduler*>(h);
  if (slot < 0 || slot >= s->max_slots || !s->slots[slot].used) return -1;
  return s->slots[slot].seq_len;
}

long long areno_sched_slot_request(void* h, int slot) {
  auto* s = static_cast<Scheduler*>(h);
  if (slot < 0 || slot >= s->max_slots || !s->slots[slot].used) return -1;
  return s->slots[slot].req_id;
}

int areno_sched_num_running(void* h) { return static_cast<Scheduler*>(h)->running; }
int areno_sched_num_waiting(void* h) { return static_cast<int>(static_cast<Scheduler*>(h)->waiting.size()); }
int areno_sched_num_free_pages(void* h) { return static_cast<int>(static_cast<Scheduler*>(h)->free_pages.size()); }

// Highest used slot index + 1 (the decode batch must cover slots [0, active_extent)).
int areno_sched_active_extent(void* h) {
  auto* s = static_cast<Scheduler*>(h);
  int ext = 0;
  for (int i = 0; i < s->max_slots; ++i)
    if (s->slots[i].used) ext = i + 1;
  return ext;
}

// Longest context among the decoding slots (tokens with KV after the planned step); 0 when none decode.
int areno_sched_max_seq_len(void* h) {
  auto* s = static_cast<Scheduler*>(h);
  int m = 0;
  for (auto& sl : s->slots)
    if (sl.used && !sl.prefilling) m = std::max(m, sl.seq_len);
  return m;
}

// Number of slots that are decoding (prompt fully prefilled).
int areno_sched_num_decoding(void* h) {
  auto* s = static_cast<Scheduler*>(h);
  int n = 0;
  for (auto& sl : s->slots)
    if (sl.used && !sl.prefilling) ++n;
  return n;
}

// Drop every waiting request (used on cancel); returns how many were dropped.
int areno_sched_clear_waiting(void* h) {
  auto* s = static_cast<Scheduler*>(h);
  const int n = static_cast<int>(s->waiting.size());
  s->waiting.clear();
  return n;
}

// ---- batch packer: padded [B, T] rows -> packed token / action index lists ---------------------
// lengths[b] valid tokens per row.  Writes token_rows/token_cols (total tokens) and action_idx
// (indices into the packed token axis of every position that predicts a next token, i.e. all but
// the last token of each row).  Returns total token count.
long long areno_pack_indices(const long long* lengths, int batch, int max_len, long long* token_rows,
                             long long* token_cols, long long* action_idx, long long* action_rows,
                             long long* n_actions_out) {
  long long t = 0, a = 0;
  for (int b = 0; b < batch; ++b) {
    long long len = lengths[b];
    if (len < 1) len = 1;
    if (len > max_len) len = max_len;
    for (long long c = 0; c < len; ++c) {
      token_rows[t] = b;
      token_cols[t] = c;
      if (c + 1 < len) {
        action_idx[a] = t;
        action_rows[a] = b;
        ++a;
      }
      ++t;
    }
  }
  *n_actions_out = a;
  return t;
}

}  // extern "C"

// Host runtime for serving: paged-KV page allocator and a continuous-batching scheduler (C ABI).
//
// The reference grows its KV cache with a tensor concatenation per step (src/models/gemma/layers.rs:29-45)
// and batches decode in fixed "slots" with a head-major cache (src/models/inkling/burn.rs:1415-1473); its
// speculative rows live in a pending region that `commit(keep)` truncates (burn.rs:381-481).  Here the cache
// is paged (16-token pages by default): a sequence owns a list of page ids, speculation appends tokens that
// `kv_truncate` rolls back, and the scheduler packs prefill chunks and decode rows of many sequences into one
// flattened batch under a token budget, admitting requests only while pages are available (the admission
// idea of src/models/inkling/budget.rs:677).
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <deque>
#include <unordered_map>
#include <vector>

namespace {

struct Seq {
  std::vector<int32_t> pages;
  int64_t len = 0;  // tokens whose K/V are in the cache
};

struct KvAlloc {
  int32_t page_size, num_pages;
  std::vector<int32_t> free_list;  // stack
  std::unordered_map<int64_t, Seq> seqs;
  int64_t peak_used = 0;
};

struct Request {
  int64_t id;
  std::vector<int32_t> prompt;
  int64_t prefilled = 0;   // prompt tokens already scheduled
  int32_t max_new = 0;
  int32_t generated = 0;
  int32_t pending = -1;    // last sampled token, to be fed at the next decode step
  bool finished = false;
  int32_t spec = 0;        // draft tokens appended to the next decode row group
  int32_t drafts[8];
  int32_t need_pages = 0;  // pages the request can grow to: prompt + max_new + 8 speculative rows (fixed at admission)
};

struct Sched {
  KvAlloc* kv;
  int32_t max_tokens;      // token budget of one step
  int32_t max_seqs;        // sequences per step
  int32_t prefill_chunk;   // longest prefill slice of one sequence in one step
  std::deque<int64_t> waiting;
  std::vector<int64_t> running;
  std::unordered_map<int64_t, Request> reqs;
  // last built batch
  std::vector<int64_t> b_seq_ids;
  std::vector<int32_t> b_q_len, b_is_decode;
};

int32_t pages_for(const KvAlloc* a, int64_t tokens) { return (int32_t)((tokens + a->page_size - 1) / a->page_size); }

}  // namespace

extern "C" {

// ----------------------------------------------------------------------------- page allocator
void* kv_create(int32_t num_pages, int32_t page_size) {
  KvAlloc* a = new KvAlloc();
  a->page_size = page_size;
  a->num_pages = num_pages;
  a->free_list.resize(num_pages);
  for (int32_t i = 0; i < num_pages; ++i) a->free_list[i] = num_pages - 1 - i;  // pop gives 0,1,2,...
  return a;
}
void kv_destroy(void* h) { delete (KvAlloc*)h; }
int32_t kv_free_pages(void* h) { return (int32_t)((KvAlloc*)h)->free_list.size(); }
int64_t kv_peak_used(void* h) { return ((KvAlloc*)h)->peak_used; }
int64_t kv_seq_len(void* h, int64_t seq) {
  auto* a = (KvAlloc*)h;
  auto it = a->seqs.find(seq);
  return it == a->seqs.end() ? -1 : it->second.len;
}

// Grow `seq` by `tokens`; allocates pages as needed.  Returns the new length, or -1 when out of pages
// (nothing is changed in that case).
int64_t kv_extend(void* h, int64_t seq, int64_t tokens) {
  auto* a = (KvAlloc*)h;
  Seq& s = a->seqs[seq];
  int32_t need = pages_for(a, s.len + tokens) - (int32_t)s.pages.size();
  if (need > (int32_t)a->free_list.size()) {
    if (s.pages.empty() && s.len == 0) a->seqs.erase(seq);
    return -1;
  }
  for (int32_t i = 0; i < need; ++i) { s.pages.push_back(a->free_list.back()); a->free_list.pop_back(); }
  s.len += tokens;
  a->peak_used = std::max<int64_t>(a->peak_used, a->num_pages - (int64_t)a->free_list.size());
  return s.len;
}

// Roll a sequence back to `new_len` tokens (speculative rows that were rejected leave no trace);
// pages that become empty go back to the free list.
int64_t kv_truncate(void* h, int64_t seq, int64_t new_len) {
  auto* a = (KvAlloc*)h;
  auto it = a->seqs.find(seq);
  if (it == a->seqs.end() || new_len > it->second.len || new_len < 0) return -1;
  Seq& s = it->second;
  int32_t keep = pages_for(a, new_len);
  while ((int32_t)s.pages.size() > keep) { a->free_list.push_back(s.pages.back()); s.pages.pop_back(); }
  s.len = new_len;
  return new_len;
}

void kv_release(void* h, int64_t seq) {
  auto* a = (KvAlloc*)h;
  auto it = a->seqs.find(seq);
  if (it == a->seqs.end()) return;
  for (auto p = it->second.pages.rbegin(); p != it->second.pages.rend(); ++p) a->free_list.push_back(*p);
  a->seqs.erase(it);
}

// Copy the page list of `seq` into out[0..max); returns the number of pages.
int32_t kv_pages(void* h, int64_t seq, int32_t* out, int32_t max) {
  auto* a = (KvAlloc*)h;
  auto it = a->seqs.find(seq);
  if (it == a->seqs.end()) return -1;
  int32_t n = (int32_t)it->second.pages.size();
  std::memcpy(out, it->second.pages.data(), sizeof(int32_t) * std::min(n, max));
  return n;
}

// Fill a [n_seqs, max_pages] table (row-major, padded with -1) and the kv lengths for a list of sequences.
int32_t kv_page_table(void* h, const int64_t* seqs, int32_t n_seqs, int32_t* table, int32_t max_pages, int32_t* kv_lens) {
  auto* a = (KvAlloc*)h;
  for (int32_t i = 0; i < n_seqs; ++i) {
    auto it = a->seqs.find(seqs[i]);
    if (it == a->seqs.end()) return -1;
    int32_t n = (int32_t)it->second.pages.size();
    if (n > max_pages) return -2;
    int32_t* row = table + (int64_t)i * max_pages;
    std::memcpy(row, it->second.pages.data(), sizeof(int32_t) * n);
    for (int32_t j = n; j < max_pages; ++j) row[j] = -1;
    kv_lens[i] = (int32_t)it->second.len;
  }
  return 0;
}

// ----------------------------------------------------------------------------- scheduler
void* sched_create(void* kv, int32_t max_tokens, int32_t max_seqs, int32_t prefill_chunk) {
  Sched* s = new Sched();
  s->kv = (KvAlloc*)kv;
  s->max_tokens = max_tokens;
  s->max_seqs = max_seqs;
  s->prefill_chunk = prefill_chunk;
  return s;
}
void sched_destroy(void* h) { delete (Sched*)h; }

// Returns 0, or -1 for a request that can never be scheduled: an empty prompt (no row to run, so it would block the head of
// the waiting queue for ever), a negative budget, or more pages than the whole pool holds.
int32_t sched_add(void* h, int64_t id, const int32_t* prompt, int32_t n, int32_t max_new) {
  Sched* s = (Sched*)h;
  if (n <= 0 || max_new < 0 || pages_for(s->kv, (int64_t)n + max_new + 8) > s->kv->num_pages) return -1;
  Request r;
  r.id = id;
  r.prompt.assign(prompt, prompt + n);
  r.max_new = max_new;
  s->reqs.emplace(id, std::move(r));
  s->waiting.push_back(id);
  return 0;
}

int32_t sched_num_waiting(void* h) { return (int32_t)((Sched*)h)->waiting.size(); }
int32_t sched_num_running(void* h) { return (int32_t)((Sched*)h)->running.size(); }

// Attach draft tokens to a running sequence: its next decode step feeds [pending, drafts...] (k+1 rows).
int32_t sched_set_drafts(void* h, int64_t id, const int32_t* drafts, int32_t k) {
  Sched* s = (Sched*)h;
  auto it = s->reqs.find(id);
  if (it == s->reqs.end() || k > 8) return -1;
  it->second.spec = k;
  std::memcpy(it->second.drafts, drafts, sizeof(int32_t) * k);
  return 0;
}

// Build the next batch.  Decode rows of running sequences go first, then prefill chunks (running ones that
// still have prompt left, then newly admitted ones) while the token budget, the sequence cap and the free
// pages allow.  Outputs (caller-allocated): token_ids/positions/seq_index [max_tokens], seq_ids/q_start/q_len/
// is_decode/sample_row [max_seqs].  sample_row[i] is the batch row whose logits give sequence i its next token,
// or -1 while its prompt is not finished.  Returns the number of sequences; *n_tokens gets the rows.
int32_t sched_next(void* h, int32_t* token_ids, int32_t* positions, int32_t* seq_index, int64_t* seq_ids,
                   int32_t* q_start, int32_t* q_len, int32_t* is_decode, int32_t* sample_row, int32_t* n_tokens) {
  Sched* s = (Sched*)h;
  KvAlloc* kv = s->kv;
  int32_t nt = 0, ns = 0;
  s->b_seq_ids.clear(); s->b_q_len.clear(); s->b_is_decode.clear();
  auto emit = [&](Request& r, const int32_t* toks, int32_t n, int64_t pos0, bool decode, bool samples) {
    q_start[ns] = nt; q_len[ns] = n; is_decode[ns] = decode ? 1 : 0; seq_ids[ns] = r.id;
    for (int32_t i = 0; i < n; ++i) { token_ids[nt] = toks[i]; positions[nt] = (int32_t)(pos0 + i); seq_index[nt] = ns; ++nt; }
    sample_row[ns] = samples ? (decode ? q_start[ns] : nt - 1) : -1;
    s->b_seq_ids.push_back(r.id); s->b_q_len.push_back(n); s->b_is_decode.push_back(decode ? 1 : 0);
    ++ns;
  };
  // 1. decode rows
  for (int64_t id : s->running) {
    Request& r = s->reqs[id];
    if (r.finished || r.prefilled < (int64_t)r.prompt.size() || r.pending < 0) continue;
    int32_t n = 1 + r.spec;
    if (ns >= s->max_seqs || nt + n > s->max_tokens) break;
    int64_t pos0 = kv_seq_len(kv, id);
    if (kv_extend(kv, id, n) < 0) break;  // out of pages: the sequence waits for the next step
    int32_t toks[9];
    toks[0] = r.pending;
    for (int32_t i = 0; i < r.spec; ++i) toks[1 + i] = r.drafts[i];
    emit(r, toks, n, pos0, true, true);
  }
  // 2. prefill chunks of running sequences
  auto prefill = [&](Request& r) -> bool {
    int64_t left = (int64_t)r.prompt.size() - r.prefilled;
    int32_t n = (int32_t)std::min<int64_t>({left, (int64_t)s->prefill_chunk, (int64_t)(s->max_tokens - nt)});
    if (n <= 0 || ns >= s->max_seqs) return false;
    int64_t pos0 = r.prefilled;
    if (kv_extend(kv, r.id, n) < 0) return false;
    bool last = (r.prefilled + n == (int64_t)r.prompt.size());
    emit(r, r.prompt.data() + r.prefilled, n, pos0, false, last);
    r.prefilled += n;
    return true;
  };
  for (int64_t id : s->running) {
    Request& r = s->reqs[id];
    if (!r.finished && r.prefilled < (int64_t)r.prompt.size()) prefill(r);
  }
  // 3. admit waiting requests.  A request is admitted only if the pages it can grow to (prompt + generation budget +
  // speculative rows) fit into the free pages that are not already PROMISED to the running requests: every running request
  // keeps a claim on need_pages - held pages, so two requests that each fit alone are not both admitted into a pool that
  // cannot hold them both, and a running sequence never finds the pool empty when it has to grow.
  int64_t promised = 0;
  for (int64_t id : s->running) {
    const Request& r = s->reqs[id];
    if (r.finished) continue;
    auto it = kv->seqs.find(id);
    const int64_t held = it == kv->seqs.end() ? 0 : (int64_t)it->second.pages.size();
    promised += std::max<int64_t>(0, (int64_t)r.need_pages - held);
  }
  while (!s->waiting.empty() && ns < s->max_seqs && nt < s->max_tokens) {
    Request& r = s->reqs[s->waiting.front()];
    const int64_t need = pages_for(kv, (int64_t)r.prompt.size() + r.max_new + 8);
    if (need > (int64_t)kv->free_list.size() - promised) break;
    const int64_t free_before = (int64_t)kv->free_list.size();
    if (!prefill(r)) break;
    r.need_pages = (int32_t)need;
    promised += need - (free_before - (int64_t)kv->free_list.size());
    s->running.push_back(r.id);
    s->waiting.pop_front();
  }
  *n_tokens = nt;
  return ns;
}

// Report the outcome of the batch for one sequence: `accepted` tokens were confirmed (1 for plain decode,
// 1..k+1 with speculation) and `next_token` is the token to feed next; the cache is rolled back to drop
// rejected rows.  `finished` marks EOS.  Returns the number of tokens generated so far.
int32_t sched_commit(void* h, int64_t id, int32_t accepted, int32_t fed_rows, int32_t next_token, int32_t finished) {
  Sched* s = (Sched*)h;
  auto it = s->reqs.find(id);
  if (it == s->reqs.end()) return -1;
  Request& r = it->second;
  if (fed_rows > accepted) {
    int64_t len = kv_seq_len(s->kv, id);
    kv_truncate(s->kv, id, len - (fed_rows - accepted));
  }
  r.generated += accepted;
  r.pending = next_token;
  r.spec = 0;
  if (finished || r.generated >= r.max_new) {
    r.finished = true;
    kv_release(s->kv, id);
    s->running.erase(std::remove(s->running.begin(), s->running.end(), id), s->running.end());
  }
  return r.generated;
}

int32_t sched_is_finished(void* h, int64_t id) {
  Sched* s = (Sched*)h;
  auto it = s->reqs.find(id);
  return it == s->reqs.end() ? -1 : (it->second.finished ? 1 : 0);
}

void sched_remove(void* h, int64_t id) {
  Sched* s = (Sched*)h;
  s->reqs.erase(id);
}

}  // extern "C"

// Implementation of the host runtime core declared in core.h.
#include "core.h"

#include <algorithm>
#include <cstring>

namespace ogb {

// ------------------------------------------------------------------------------------------
// BlockPool
// ------------------------------------------------------------------------------------------
BlockPool::BlockPool(int num_pages) : ref_(num_pages, 0), hash_of_(num_pages, 0), in_evictable_(num_pages, 0) {
  free_.reserve(num_pages);
  for (int i = num_pages - 1; i >= 0; --i) free_.push_back(i);  // pop_back hands out page 0 first
}

void BlockPool::add_pages(int n) {
  if (n <= 0) return;
  const int old = num_pages();
  ref_.resize(old + n, 0);
  hash_of_.resize(old + n, 0);
  in_evictable_.resize(old + n, 0);
  // the free list hands out from its back: put the new ids at the front so existing free pages are reused first
  std::vector<int> fresh;
  fresh.reserve(free_.size() + n);
  for (int i = old + n - 1; i >= old; --i) fresh.push_back(i);
  fresh.insert(fresh.end(), free_.begin(), free_.end());
  free_.swap(fresh);
}

int BlockPool::allocate() {
  int page = -1;
  if (!free_.empty()) {
    page = free_.back();
    free_.pop_back();
  } else {
    while (!evictable_.empty()) {
      int cand = evictable_.front();
      evictable_.pop_front();
      if (!in_evictable_[cand] || ref_[cand] != 0) continue;  // stale entry
      in_evictable_[cand] = 0;
      --evictable_live_;
      page = cand;
      break;
    }
    if (page < 0) return -1;
    if (hash_of_[page] != 0) {
      auto it = by_hash_.find(hash_of_[page]);
      if (it != by_hash_.end() && it->second == page) by_hash_.erase(it);
      hash_of_[page] = 0;
    }
  }
  ref_[page] = 1;
  return page;
}

void BlockPool::release(int page) {
  if (page < 0 || page >= num_pages() || ref_[page] <= 0) return;
  if (--ref_[page] > 0) return;
  if (hash_of_[page] != 0) {
    evictable_.push_back(page);
    if (!in_evictable_[page]) ++evictable_live_;
    in_evictable_[page] = 1;
  } else {
    free_.push_back(page);
  }
}

uint64_t BlockPool::chain_hash(uint64_t parent, const int32_t* tokens, int n) {
  uint64_t h = parent ^ 0x9E3779B97F4A7C15ull;
  for (int i = 0; i < n; ++i) {
    h ^= static_cast<uint32_t>(tokens[i]) + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h *= 0xff51afd7ed558ccdull;
    h ^= h >> 33;
  }
  return h == 0 ? 1 : h;
}

int BlockPool::lookup(uint64_t hash) {
  ++lookups_;
  auto it = by_hash_.find(hash);
  if (it == by_hash_.end()) return -1;
  const int page = it->second;
  if (ref_[page] == 0 && in_evictable_[page]) {  // leaves the LRU lazily (stale deque entry is skipped)
    in_evictable_[page] = 0;
    --evictable_live_;
  }
  ++ref_[page];
  ++hits_;
  return page;
}

void BlockPool::publish(int page, uint64_t hash) {
  if (hash_of_[page] != 0) return;
  if (by_hash_.count(hash)) return;  // another page already serves this prefix
  hash_of_[page] = hash;
  by_hash_[hash] = page;
}

bool BlockPool::unpublish(int page) {
  // only a cached page that nobody references can leave the cache without a holder noticing
  if (page < 0 || page >= num_pages() || hash_of_[page] == 0 || ref_[page] != 0) return false;
  auto it = by_hash_.find(hash_of_[page]);
  if (it != by_hash_.end() && it->second == page) by_hash_.erase(it);
  hash_of_[page] = 0;
  if (in_evictable_[page]) {   // its deque entry goes stale and is skipped by allocate()
    in_evictable_[page] = 0;
    --evictable_live_;
  }
  free_.push_back(page);
  return true;
}

void BlockPool::reset_prefix_cache() {
  for (int p : evictable_) {
    if (in_evictable_[p] && ref_[p] == 0) {
      in_evictable_[p] = 0;
      free_.push_back(p);
    }
  }
  evictable_.clear();
  evictable_live_ = 0;
  by_hash_.clear();
  std::fill(hash_of_.begin(), hash_of_.end(), 0);
}

// ------------------------------------------------------------------------------------------
// Core
// ------------------------------------------------------------------------------------------
static PlanLayout make_layout(const CoreConfig& c) {
  PlanLayout l{};
  int o = 32;
  auto take = [&](int n) { int at = o; o += n; return at; };
  l.header = 0;
  l.token_ids = take(c.max_tokens_per_step);
  l.positions = take(c.max_tokens_per_step);
  l.slots = take(c.max_tokens_per_step);
  l.seq_slot = take(c.max_seqs);
  l.ctx_len = take(c.max_seqs);
  l.cu_q = take(c.max_seqs + 1);
  l.page_table = take(c.max_seqs * c.max_pages_per_seq);
  l.max_tiles = c.max_tokens_per_step / 64 + c.max_seqs + 1;
  l.tile_seq = take(l.max_tiles);
  l.tile_q0 = take(l.max_tiles);
  l.max_rows = c.max_seqs * (1 + (c.max_draft_tokens > 0 ? c.max_draft_tokens : 0));
  l.logit_rows = take(l.max_rows);
  l.temperature = take(l.max_rows);
  l.top_k = take(l.max_rows);
  l.top_p = take(l.max_rows);
  l.min_p = take(l.max_rows);
  l.uniform = take(l.max_rows);
  l.logit_seq = take(l.max_rows);
  l.copy_src = take(c.max_seqs);
  l.copy_dst = take(c.max_seqs);
  l.max_swap = c.max_seqs * c.max_pages_per_seq;
  if (c.num_host_pages == 0) l.max_swap = 1;
  l.swap_out_dev = take(l.max_swap);
  l.swap_out_host = take(l.max_swap);
  l.swap_in_dev = take(l.max_swap);
  l.swap_in_host = take(l.max_swap);
  l.max_runs = 2 * c.max_seqs + 4;
  l.move_runs = take(2 * l.max_runs);
  l.total_words = o;
  return l;
}

Core::Core(const CoreConfig& cfg) : cfg_(cfg), layout_(make_layout(cfg)), pool_(cfg.num_pages) {
  for (int i = cfg.num_host_pages - 1; i >= 0; --i) host_free_.push_back(i);
}

Sequence* Core::find(int64_t id) {
  auto it = seqs_.find(id);
  return it == seqs_.end() ? nullptr : &it->second;
}
const Sequence* Core::find(int64_t id) const {
  auto it = seqs_.find(id);
  return it == seqs_.end() ? nullptr : &it->second;
}

static uint64_t splitmix64(uint64_t& x) {
  uint64_t z = (x += 0x9E3779B97F4A7C15ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

float Core::next_uniform(Sequence& s) {
  const uint64_t r = splitmix64(s.rng_state);
  return static_cast<float>(r >> 40) * (1.0f / 16777216.0f);  // 24 random bits -> [0, 1)
}

int64_t Core::add_request(const int32_t* prompt, int n, int max_new_tokens, const SamplingParams& sp, int priority,
                          int tenant, bool ignore_eos, const int32_t* stop_ids, int n_stop) {
  if (n <= 0 || max_new_tokens < 0) return -1;
  const int max_len = cfg_.max_pages_per_seq * kPageTokens;
  if (n + max_new_tokens > max_len) {
    if (n >= max_len) return -2;  // prompt alone does not fit a page table row
    max_new_tokens = max_len - n; // admission capping, like the reference's GenerationBudgetCap
  }
  Sequence s;
  s.id = next_id_++;
  s.tokens.assign(prompt, prompt + n);
  s.prompt_len = n;
  s.max_new_tokens = max_new_tokens;
  s.sampling = sp;
  s.rng_state = sp.seed ? sp.seed : (0x1234567ull + static_cast<uint64_t>(s.id) * 0x9E3779B97F4A7C15ull);
  s.priority = priority;
  s.tenant = tenant;
  s.arrival = clock_++;
  s.ignore_eos = ignore_eos;
  if (stop_ids && n_stop > 0) s.stop_ids.assign(stop_ids, stop_ids + n_stop);
  const int64_t id = s.id;
  seqs_.emplace(id, std::move(s));
  waiting_.push_back(id);
  return id;
}

void Core::free_pages(Sequence& s, bool publish_prefix) {
  if (publish_prefix) publish_full_pages(s);
  for (int p : s.pages) if (p >= 0) pool_.release(p);
  s.pages.clear();
  s.trim_end = 0;
}

void Core::set_window(int window, int sink_tokens) {
  window_ = std::max(window, 0);
  sink_pages_ = window_ > 0 ? (std::max(sink_tokens, 0) + kPageTokens - 1) / kPageTokens : 0;
}

int Core::released_pages(int64_t seq_id) const {
  const Sequence* s = find(seq_id);
  if (!s) return -1;
  int n = 0;
  for (int p : s->pages) n += p < 0 ? 1 : 0;
  return n;
}

// The next query of `s` sits at position num_computed and sees keys above num_computed - window; a rejected draft can
// pull num_computed back by at most max_draft_tokens, and one more page of slack keeps ordinary session rewinds cheap.
void Core::trim_window(Sequence& s) {
  if (window_ <= 0) return;
  const int first_needed = s.num_computed - window_ - cfg_.max_draft_tokens - kPageTokens;
  const int hi = std::min(first_needed / kPageTokens, static_cast<int>(s.pages.size()));
  const int lo = std::max(sink_pages_, s.trim_end);
  if (first_needed <= 0 || hi <= lo) return;
  for (int i = lo; i < hi; ++i) {
    if (s.pages[i] >= 0) { pool_.release(s.pages[i]); s.pages[i] = -1; }
  }
  s.trim_end = hi;
}

void Core::publish_full_pages(Sequence& s) {
  if (!cfg_.enable_prefix_cache) return;
  const int full = std::min(s.num_computed, static_cast<int>(s.tokens.size())) / kPageTokens;
  uint64_t h = 0;
  for (int i = 0; i < full && i < static_cast<int>(s.pages.size()); ++i) {
    h = BlockPool::chain_hash(h, s.tokens.data() + i * kPageTokens, kPageTokens);
    if (s.pages[i] >= 0) pool_.publish(s.pages[i], h);
  }
}

void Core::try_prefix_attach(Sequence& s) {
  if (!cfg_.enable_prefix_cache || !s.pages.empty()) return;
  // never serve the whole prompt from cache: the last token must run to produce logits
  const int max_full = (static_cast<int>(s.tokens.size()) - 1) / kPageTokens;
  uint64_t h = 0;
  int matched = 0;
  for (int i = 0; i < max_full; ++i) {
    h = BlockPool::chain_hash(h, s.tokens.data() + i * kPageTokens, kPageTokens);
    const int page = pool_.lookup(h);
    if (page < 0) break;
    s.pages.push_back(page);
    ++matched;
  }
  s.num_computed = matched * kPageTokens;
  s.num_cached_prefix = s.num_computed;
}

bool Core::ensure_pages(Sequence& s, int new_len, std::vector<std::pair<int, int>>& copies) {
  const int need = (new_len + kPageTokens - 1) / kPageTokens;
  if (need > cfg_.max_pages_per_seq) return false;
  // copy-on-write: the page that receives the next token must be exclusively owned
  const int write_page = s.num_computed / kPageTokens;
  if (write_page < static_cast<int>(s.pages.size()) && pool_.refcount(s.pages[write_page]) > 1 &&
      (s.num_computed % kPageTokens) != 0) {
    const int fresh = pool_.allocate();
    if (fresh < 0) return false;
    copies.emplace_back(s.pages[write_page], fresh);
    move_kinds_.push_back(0);
    pool_.release(s.pages[write_page]);
    s.pages[write_page] = fresh;
  }
  const int have = static_cast<int>(s.pages.size());
  if (need - have > pool_.num_free()) return false;
  for (int i = have; i < need; ++i) {
    const int p = pool_.allocate();
    if (p < 0) return false;  // cannot happen after the check above
    s.pages.push_back(p);
  }
  return true;
}

bool Core::preempt_one(Sequence* keep, std::vector<std::pair<int, int>>& swap_out) {
  // victim: lowest priority, then latest arrival, among running sequences other than `keep`
  int victim_idx = -1;
  for (int i = 0; i < static_cast<int>(running_.size()); ++i) {
    Sequence* c = find(running_[i]);
    if (!c || c == keep) continue;
    if (victim_idx < 0) { victim_idx = i; continue; }
    Sequence* v = find(running_[victim_idx]);
    if (c->priority < v->priority || (c->priority == v->priority && c->arrival > v->arrival)) victim_idx = i;
  }
  if (victim_idx < 0) return false;
  Sequence& v = *find(running_[victim_idx]);
  running_.erase(running_.begin() + victim_idx);
  ++preemptions_;
  if (v.num_draft > 0) {  // unverified drafts never survive a preemption
    v.tokens.resize(v.tokens.size() - v.num_draft);
    v.num_draft = 0;
  }
  v.scheduled = 0;
  v.samples_this_step = false;
  const int used_pages = (v.num_computed + kPageTokens - 1) / kPageTokens;
  if (cfg_.preempt == PreemptMode::Swap && static_cast<int>(host_free_.size()) >= used_pages && used_pages > 0) {
    v.host_pages.clear();
    for (int i = 0; i < used_pages; ++i) {
      if (v.pages[i] < 0) { v.host_pages.push_back(-1); continue; }   // released under the sliding window: nothing to save
      const int hp = host_free_.back();
      host_free_.pop_back();
      v.host_pages.push_back(hp);
      swap_out.emplace_back(v.pages[i], hp);
      move_kinds_.push_back(1);
    }
    for (int p : v.pages) if (p >= 0) pool_.release(p);
    v.pages.clear();
    v.status = SeqStatus::Swapped;
    swapped_.push_back(v.id);
  } else {
    free_pages(v, true);
    v.num_computed = 0;
    v.status = SeqStatus::Waiting;
    waiting_.push_front(v.id);
  }
  return true;
}

std::vector<int64_t> Core::waiting_order() {
  std::vector<int64_t> order(waiting_.begin(), waiting_.end());
  if (cfg_.policy == Policy::Priority) {
    std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) {
      const Sequence *sa = find(a), *sb = find(b);
      if (sa->priority != sb->priority) return sa->priority > sb->priority;
      return sa->arrival < sb->arrival;
    });
  } else if (cfg_.policy == Policy::FairShare) {
    std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) {
      const Sequence *sa = find(a), *sb = find(b);
      const int64_t ta = tenant_served_[sa->tenant], tb = tenant_served_[sb->tenant];
      if (ta != tb) return ta < tb;  // least-served tenant first
      return sa->arrival < sb->arrival;
    });
  }
  return order;
}

int Core::build_step(int32_t* plan) {
  const PlanLayout& L = layout_;
  std::memset(plan, 0, sizeof(int32_t) * 32);
  ++step_id_;
  move_kinds_.clear();
  std::vector<std::pair<int, int>> copies, swap_out, swap_in;
  int budget = cfg_.max_tokens_per_step;

  struct Item { Sequence* s; int n; };
  std::vector<Item> decode_items, prefill_items;

  // 1. sequences already running: decode rows take one token, unfinished prompts take a chunk
  for (size_t i = 0; i < running_.size();) {
    Sequence* s = find(running_[i]);
    int remaining = static_cast<int>(s->tokens.size()) - s->num_computed;
    s->num_draft = 0;
    if (remaining == 1 && !s->draft.empty() && cfg_.max_draft_tokens > 0) {
      // speculative verification: feed the last token and the drafts as one short chunk
      int k = std::min<int>(static_cast<int>(s->draft.size()), cfg_.max_draft_tokens);
      const int generated = static_cast<int>(s->tokens.size()) - s->prompt_len;
      k = std::min(k, std::max(0, s->max_new_tokens - generated - 1));
      k = std::min(k, cfg_.max_pages_per_seq * kPageTokens - static_cast<int>(s->tokens.size()));
      if (k > 0 && 1 + k <= budget) {
        s->tokens.insert(s->tokens.end(), s->draft.begin(), s->draft.begin() + k);
        s->num_draft = k;
        remaining = 1 + k;
      }
      s->draft.clear();
    }
    int n = std::min({remaining, budget, remaining > 1 ? cfg_.prefill_chunk : 1});
    if (s->num_draft > 0) n = remaining;
    if (n <= 0) { s->scheduled = 0; ++i; continue; }
    bool ok = ensure_pages(*s, s->num_computed + n, copies);
    while (!ok) {
      if (!preempt_one(s, swap_out)) break;
      ok = ensure_pages(*s, s->num_computed + n, copies);
    }
    // preempt_one may have removed an element before position i
    size_t pos = std::find(running_.begin(), running_.end(), s->id) - running_.begin();
    i = pos;
    if (!ok) {
      // alone and still out of pages: this sequence can never advance; fail it
      finish(*s, FinishReason::Error);
      continue;
    }
    s->scheduled = n;
    budget -= n;
    (remaining == 1 ? decode_items : prefill_items).push_back({s, n});
    ++i;
  }
  // (a preempted speculative sequence drops its drafts: see preempt_one)
  // drop items whose sequence was preempted after being scheduled
  auto still_running = [&](const Item& it) { return it.s->status == SeqStatus::Running && it.s->scheduled > 0; };
  decode_items.erase(std::remove_if(decode_items.begin(), decode_items.end(), [&](const Item& it) { return !still_running(it); }),
                     decode_items.end());
  prefill_items.erase(std::remove_if(prefill_items.begin(), prefill_items.end(), [&](const Item& it) { return !still_running(it); }),
                      prefill_items.end());

  // 2. swapped sequences come back first (they hold progress), then new admissions
  while (!swapped_.empty() && budget > 0 && static_cast<int>(running_.size()) < cfg_.max_seqs && swap_out.empty()) {
    Sequence* s = find(swapped_.front());
    const int used_pages = static_cast<int>(s->host_pages.size());
    if (used_pages + 1 > pool_.num_free()) break;
    for (int i = 0; i < used_pages; ++i) {
      if (s->host_pages[i] < 0) { s->pages.push_back(-1); continue; }
      const int p = pool_.allocate();
      s->pages.push_back(p);
      swap_in.emplace_back(p, s->host_pages[i]);
      move_kinds_.push_back(2);
      host_free_.push_back(s->host_pages[i]);
    }
    s->host_pages.clear();
    swapped_.pop_front();
    s->status = SeqStatus::Running;
    running_.push_back(s->id);
    const int remaining = static_cast<int>(s->tokens.size()) - s->num_computed;
    const int n = std::min({remaining, budget, remaining > 1 ? cfg_.prefill_chunk : 1});
    if (n > 0 && ensure_pages(*s, s->num_computed + n, copies)) {
      s->scheduled = n;
      budget -= n;
      (remaining == 1 ? decode_items : prefill_items).push_back({s, n});
    }
  }
  if (swapped_.empty() && swap_out.empty()) {
    for (int64_t id : waiting_order()) {
      if (budget <= 0 || static_cast<int>(running_.size()) >= cfg_.max_seqs) break;
      Sequence* s = find(id);
      if (s->pages.empty() && s->num_computed == 0) try_prefix_attach(*s);
      const int remaining = static_cast<int>(s->tokens.size()) - s->num_computed;
      int n = std::min({remaining, budget, cfg_.prefill_chunk});
      if (n <= 0) break;
      // keep one page of headroom per running sequence so decode rows are not starved next step
      const int need = (s->num_computed + n + kPageTokens - 1) / kPageTokens - static_cast<int>(s->pages.size());
      if (need + static_cast<int>(running_.size()) > pool_.num_free()) {
        if (s->num_cached_prefix > 0 && s->num_computed == s->num_cached_prefix) {  // give the cached pages back
          free_pages(*s, false);
          s->num_computed = 0;
          s->num_cached_prefix = 0;
        }
        break;
      }
      if (!ensure_pages(*s, s->num_computed + n, copies)) break;
      waiting_.erase(std::find(waiting_.begin(), waiting_.end(), id));
      s->status = SeqStatus::Running;
      running_.push_back(id);
      s->scheduled = n;
      budget -= n;
      tenant_served_[s->tenant] += n;
      (remaining == 1 ? decode_items : prefill_items).push_back({s, n});
    }
  }

  // 3. optional rounding of the step size: shrink the last prefill chunk so T % token_multiple == 0
  int total = 0;
  for (auto& it : decode_items) total += it.n;
  for (auto& it : prefill_items) total += it.n;
  if (cfg_.token_multiple > 1 && !prefill_items.empty()) {
    int excess = total % cfg_.token_multiple;
    for (int i = static_cast<int>(prefill_items.size()) - 1; i >= 0 && excess > 0; --i) {
      Item& it = prefill_items[i];
      const int remaining = static_cast<int>(it.s->tokens.size()) - it.s->num_computed;
      const bool completes = (it.n == remaining);
      if (it.s->num_draft > 0) continue;  // a verification chunk is all-or-nothing
      int cut = std::min(excess, it.n - 1);
      if (completes && cut > 0 && it.n - cut < 1) cut = 0;
      if (cut > 0) { it.n -= cut; it.s->scheduled = it.n; excess -= cut; total -= cut; }
    }
  }

  // 4. emit the plan: decode rows first, then prefill chunks
  int t = 0, row = 0, nlog = 0, ntiles = 0, max_ctx = 0;
  step_rows_.clear();
  step_seqs_.clear();
  auto emit = [&](Sequence* s, int n, bool is_prefill, int prefill_token_base) {
    const int start = s->num_computed;
    for (int j = 0; j < n; ++j) {
      const int pos = start + j;
      plan[L.token_ids + t + j] = s->tokens[pos];
      plan[L.positions + t + j] = pos;
      plan[L.slots + t + j] = s->pages[pos / kPageTokens] * kPageTokens + pos % kPageTokens;
    }
    const int ctx = start + n;
    max_ctx = std::max(max_ctx, ctx);
    plan[L.ctx_len + row] = ctx;
    plan[L.seq_slot + row] = static_cast<int32_t>(s->id & 0x7fffffff);
    int32_t* pt = plan + L.page_table + static_cast<size_t>(row) * cfg_.max_pages_per_seq;
    const int np = static_cast<int>(s->pages.size());
    for (int j = 0; j < np; ++j) pt[j] = s->pages[j];
    if (is_prefill) {
      const int prow = row - static_cast<int>(decode_items.size());
      plan[L.cu_q + prow] = t - prefill_token_base;
      plan[L.cu_q + prow + 1] = t - prefill_token_base + n;
      // longest tiles first: the last query block of a chunk attends to the most keys
      for (int q0 = ((n - 1) / 64) * 64; q0 >= 0; q0 -= 64) {
        plan[L.tile_seq + ntiles] = prow;
        plan[L.tile_q0 + ntiles] = q0;
        ++ntiles;
      }
    }
    const bool completes = (ctx == static_cast<int>(s->tokens.size()));
    s->samples_this_step = completes;
    if (completes) {
      // one logit row for the last position, or one per fed position when drafts are being verified
      const int first = s->num_draft > 0 ? 0 : n - 1;
      for (int j = first; j < n && nlog < L.max_rows; ++j) {
        plan[L.logit_rows + nlog] = t + j;
        plan[L.logit_seq + nlog] = static_cast<int32_t>(s->id & 0x7fffffff);
        float tmp = s->sampling.temperature;
        std::memcpy(&plan[L.temperature + nlog], &tmp, 4);
        plan[L.top_k + nlog] = s->sampling.top_k;
        tmp = s->sampling.top_p;
        std::memcpy(&plan[L.top_p + nlog], &tmp, 4);
        tmp = s->sampling.min_p;
        std::memcpy(&plan[L.min_p + nlog], &tmp, 4);
        tmp = (s->sampling.temperature > 0.f) ? next_uniform(*s) : 0.f;
        std::memcpy(&plan[L.uniform + nlog], &tmp, 4);
        step_rows_.push_back(s->id);
        ++nlog;
      }
    }
    step_seqs_.push_back(s->id);
    t += n;
    ++row;
  };
  for (auto& it : decode_items) emit(it.s, it.n, false, 0);
  const int prefill_base = t;
  for (auto& it : prefill_items) emit(it.s, it.n, true, prefill_base);

  int ncopy = 0;
  for (auto& c : copies) {
    if (ncopy >= cfg_.max_seqs) break;
    plan[L.copy_src + ncopy] = c.first;
    plan[L.copy_dst + ncopy] = c.second;
    ++ncopy;
  }
  int nso = 0, nsi = 0;
  for (auto& c : swap_out) { if (nso < L.max_swap) { plan[L.swap_out_dev + nso] = c.first; plan[L.swap_out_host + nso] = c.second; ++nso; } }
  for (auto& c : swap_in) { if (nsi < L.max_swap) { plan[L.swap_in_dev + nsi] = c.first; plan[L.swap_in_host + nsi] = c.second; ++nsi; } }

  // The page moves must run in the order they were decided: a page that a victim frees by swapping out can be
  // handed out again as the target of a later copy, and a page that was the target of a copy can belong to a
  // sequence preempted later in the same step.  Runs of one kind are kept together; the lists above are in
  // decision order within each kind.
  int nruns = 0;
  {
    int emitted[3] = {0, 0, 0};
    const int limit[3] = {ncopy, nso, nsi};
    for (size_t i = 0; i < move_kinds_.size(); ++i) {
      const int k = move_kinds_[i];
      if (emitted[k] >= limit[k]) continue;   // an entry the list had no room for
      ++emitted[k];
      if (nruns > 0 && plan[L.move_runs + 2 * (nruns - 1)] == k) {
        ++plan[L.move_runs + 2 * (nruns - 1) + 1];
      } else if (nruns < L.max_runs) {
        plan[L.move_runs + 2 * nruns] = k;
        plan[L.move_runs + 2 * nruns + 1] = 1;
        ++nruns;
      }
    }
  }
  plan[kHdrNumMoveRuns] = nruns;
  plan[kHdrNumTokens] = t;
  plan[kHdrNumDecode] = static_cast<int>(decode_items.size());
  plan[kHdrNumPrefillSeqs] = static_cast<int>(prefill_items.size());
  plan[kHdrNumTiles] = ntiles;
  plan[kHdrNumLogitRows] = nlog;
  plan[kHdrNumCopies] = ncopy;
  plan[kHdrNumSwapOut] = nso;
  plan[kHdrNumSwapIn] = nsi;
  plan[kHdrNumPrefillTokens] = t - prefill_base;
  plan[kHdrMaxCtx] = max_ctx;
  plan[kHdrNumPreempted] = static_cast<int>(preemptions_ & 0x7fffffff);
  plan[kHdrStepId] = static_cast<int>(step_id_ & 0x7fffffff);
  return t;
}

void Core::finish(Sequence& s, FinishReason why) {
  s.finish = why;
  s.status = SeqStatus::Finished;
  s.scheduled = 0;
  free_pages(s, why != FinishReason::Error);
  for (int hp : s.host_pages) if (hp >= 0) host_free_.push_back(hp);
  s.host_pages.clear();
  running_.erase(std::remove(running_.begin(), running_.end(), s.id), running_.end());
  waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), s.id), waiting_.end());
  swapped_.erase(std::remove(swapped_.begin(), swapped_.end(), s.id), swapped_.end());
}

int Core::commit_step(const int32_t* sampled, int n, StepEvent* events, int max_events) {
  int ne = 0;
  // advance every scheduled sequence
  for (int64_t id : step_seqs_) {
    Sequence* s = find(id);
    if (!s || s->status != SeqStatus::Running) continue;
    s->num_computed += s->scheduled;
    s->scheduled = 0;
  }
  const int rows = std::min(n, static_cast<int>(step_rows_.size()));
  auto push_token = [&](Sequence* s, int32_t tok) -> bool {  // returns true when the sequence finished
    s->tokens.push_back(tok);
    const int generated = static_cast<int>(s->tokens.size()) - s->prompt_len;
    FinishReason why = FinishReason::None;
    if (!s->ignore_eos && cfg_.eos_token >= 0 && tok == cfg_.eos_token) why = FinishReason::Stop;
    for (int32_t st : s->stop_ids) if (tok == st) why = FinishReason::Stop;
    if (why == FinishReason::None && generated >= s->max_new_tokens) why = FinishReason::Length;
    if (why != FinishReason::None) finish(*s, why);
    if (ne < max_events) events[ne++] = StepEvent{s->id, tok, static_cast<int32_t>(why)};
    return why != FinishReason::None;
  };
  for (int r = 0; r < rows;) {
    Sequence* s = find(step_rows_[r]);
    int group = 1;
    while (r + group < rows && step_rows_[r + group] == step_rows_[r]) ++group;
    if (!s || s->status != SeqStatus::Running || !s->samples_this_step) { r += group; continue; }
    s->samples_this_step = false;
    if (s->num_draft > 0 && group == s->num_draft + 1) {
      // tokens = [... last, d0 .. d(k-1)]; sampled[r + j] follows position (last + j)
      const int k = s->num_draft;
      const int base = static_cast<int>(s->tokens.size()) - k;   // index of d0
      int a = 0;
      while (a < k && s->tokens[base + a] == sampled[r + a]) ++a;
      ++spec_steps_;
      spec_proposed_ += k;
      spec_accepted_ += a;
      std::vector<int32_t> accepted(s->tokens.begin() + base, s->tokens.begin() + base + a);
      s->tokens.resize(base);
      s->num_draft = 0;
      // K/V of the last token and of the accepted drafts are valid; everything after is rewound
      s->num_computed = base + a;
      const int keep_pages = (s->num_computed + kPageTokens - 1) / kPageTokens;
      while (static_cast<int>(s->pages.size()) > keep_pages) {
        if (s->pages.back() >= 0) pool_.release(s->pages.back());
        s->pages.pop_back();
      }
      bool done = false;
      for (int j = 0; j < a && !done; ++j) done = push_token(s, accepted[j]);
      if (done) {
        // finished inside the accepted run: later accepted tokens are dropped with the sequence
      } else {
        push_token(s, sampled[r + a]);
      }
    } else {
      push_token(s, sampled[r + group - 1]);
    }
    r += group;
  }
  if (window_ > 0) {
    for (int64_t id : step_seqs_) {
      Sequence* s = find(id);
      if (s && s->status == SeqStatus::Running) trim_window(*s);
    }
  }
  step_rows_.clear();
  step_seqs_.clear();
  return ne;
}

bool Core::cancel(int64_t seq_id) {
  Sequence* s = find(seq_id);
  if (!s || s->status == SeqStatus::Finished) return false;
  finish(*s, FinishReason::Cancelled);
  return true;
}

int64_t Core::fork(int64_t seq_id) {
  Sequence* s = find(seq_id);
  if (!s) return -1;
  Sequence c = *s;
  c.id = next_id_++;
  c.arrival = clock_++;
  c.host_pages.clear();
  c.scheduled = 0;
  c.samples_this_step = false;
  c.rng_state ^= 0xD1B54A32D192ED03ull * static_cast<uint64_t>(c.id);
  for (int p : c.pages) if (p >= 0) pool_.retain(p);
  if (s->status == SeqStatus::Swapped) {  // a swapped parent has no device pages to share
    c.pages.clear();
    c.trim_end = 0;
    c.num_computed = 0;
    c.status = SeqStatus::Waiting;
  }
  if (c.status == SeqStatus::Finished) { c.status = SeqStatus::Waiting; c.finish = FinishReason::None; }
  const int64_t id = c.id;
  const SeqStatus st = c.status;
  seqs_.emplace(id, std::move(c));
  if (st == SeqStatus::Running) running_.push_back(id); else waiting_.push_back(id);
  return id;
}

bool Core::swap_state(int64_t a, int64_t b) {
  Sequence* sa = find(a);
  Sequence* sb = find(b);
  if (!sa || !sb || a == b) return false;
  std::swap(*sa, *sb);
  std::swap(sa->id, sb->id);
  std::swap(sa->arrival, sb->arrival);
  for (Sequence* s : {sa, sb}) {          // queue membership follows the status each id now has
    running_.erase(std::remove(running_.begin(), running_.end(), s->id), running_.end());
    waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), s->id), waiting_.end());
    swapped_.erase(std::remove(swapped_.begin(), swapped_.end(), s->id), swapped_.end());
    if (s->status == SeqStatus::Running) running_.push_back(s->id);
    else if (s->status == SeqStatus::Waiting) waiting_.push_back(s->id);
    else if (s->status == SeqStatus::Swapped) swapped_.push_back(s->id);
  }
  return true;
}

bool Core::rewind(int64_t seq_id, int new_len) {
  Sequence* s = find(seq_id);
  if (!s || new_len < 1 || new_len > static_cast<int>(s->tokens.size())) return false;
  // keys released under the sliding window cannot come back into view
  if (s->trim_end > sink_pages_ && std::min(new_len, s->num_computed) - window_ < s->trim_end * kPageTokens) return false;
  s->tokens.resize(new_len);
  if (s->prompt_len > new_len) s->prompt_len = new_len;
  // the last kept token must be re-run to produce logits unless its successor is about to be fed
  if (s->num_computed > new_len) s->num_computed = new_len;
  const int keep_pages = (s->num_computed + kPageTokens - 1) / kPageTokens;
  while (static_cast<int>(s->pages.size()) > keep_pages) {
    if (s->pages.back() >= 0) pool_.release(s->pages.back());
    s->pages.pop_back();
  }
  return true;
}

bool Core::set_draft(int64_t seq_id, const int32_t* tokens, int k) {
  Sequence* s = find(seq_id);
  if (!s || s->status == SeqStatus::Finished || k < 0) return false;
  s->draft.assign(tokens, tokens + k);
  return true;
}

bool Core::append_tokens(int64_t seq_id, const int32_t* tokens, int n) {
  Sequence* s = find(seq_id);
  if (!s || n < 0 || s->status == SeqStatus::Finished) return false;
  if (static_cast<int>(s->tokens.size()) + n > cfg_.max_pages_per_seq * kPageTokens) return false;
  s->tokens.insert(s->tokens.end(), tokens, tokens + n);
  s->prompt_len = static_cast<int>(s->tokens.size());   // the generation budget counts from here
  s->draft.clear();
  return true;
}

int Core::seq_pages(int64_t seq_id, int32_t* out, int cap) const {
  const Sequence* s = find(seq_id);
  if (!s) return -1;
  const int used = std::min(static_cast<int>(s->pages.size()), (s->num_computed + kPageTokens - 1) / kPageTokens);
  const int n = std::min(cap, used);
  for (int i = 0; i < n; ++i) out[i] = s->pages[i];
  return n;
}

int Core::prefix_adopt(const int32_t* tokens, int n_tokens, int32_t* out_pages, int cap) {
  if (!cfg_.enable_prefix_cache) return 0;
  const int full = std::min(cap, n_tokens / kPageTokens);
  uint64_t h = 0;
  int served = 0;
  // Adopted pages stay referenced until the loop ends: released at once they would be the first candidates for
  // eviction by the next allocation of this very call, and a pool smaller than the prefix would hand the same
  // page out twice.
  std::vector<int> held;
  for (int i = 0; i < full; ++i) {
    h = BlockPool::chain_hash(h, tokens + i * kPageTokens, kPageTokens);
    if (pool_.contains(h)) {
      const int page = pool_.peek(h);
      pool_.retain(page);                 // referenced, so it cannot be evicted below (not a request hit: no statistics)
      held.push_back(page);
      out_pages[i] = -1;
    } else {
      const int page = pool_.allocate();
      if (page < 0) break;
      pool_.publish(page, h);
      held.push_back(page);
      out_pages[i] = page;
    }
    ++served;
  }
  for (int page : held) pool_.release(page);   // cached and unreferenced: the next admission with this prefix retains them
  return served;
}

int Core::prefix_unpublish(const int32_t* pages, int n) {
  int done = 0;
  for (int i = 0; i < n; ++i) done += pool_.unpublish(pages[i]) ? 1 : 0;
  return done;
}

int Core::prefix_peek(const int32_t* tokens, int n_tokens, int32_t* out_pages, int cap) const {
  if (!cfg_.enable_prefix_cache) return 0;
  const int full = std::min(cap, n_tokens / kPageTokens);
  uint64_t h = 0;
  int n = 0;
  for (; n < full; ++n) {
    h = BlockPool::chain_hash(h, tokens + n * kPageTokens, kPageTokens);
    const int page = pool_.peek(h);
    if (page < 0) break;
    out_pages[n] = page;
  }
  return n;
}

int Core::seq_len(int64_t seq_id) const {
  const Sequence* s = find(seq_id);
  return s ? static_cast<int>(s->tokens.size()) : -1;
}

int Core::seq_computed(int64_t seq_id) const {
  const Sequence* s = find(seq_id);
  return s ? s->num_computed : -1;
}

int Core::seq_tokens(int64_t seq_id, int32_t* out, int cap) const {
  const Sequence* s = find(seq_id);
  if (!s) return -1;
  const int n = std::min(cap, static_cast<int>(s->tokens.size()));
  std::memcpy(out, s->tokens.data(), sizeof(int32_t) * n);
  return static_cast<int>(s->tokens.size());
}

void Core::release(int64_t seq_id) {
  Sequence* s = find(seq_id);
  if (!s) return;
  if (s->status != SeqStatus::Finished) finish(*s, FinishReason::Cancelled);
  seqs_.erase(seq_id);
}

}  // namespace ogb

// ------------------------------------------------------------------------------------------
// C ABI for ctypes
// ------------------------------------------------------------------------------------------
using namespace ogb;

extern "C" {

void* ogb_core_create(int num_pages, int num_host_pages, int max_seqs, int max_tokens_per_step, int max_pages_per_seq,
                      int prefill_chunk, int token_multiple, int policy, int preempt_mode, int enable_prefix_cache,
                      int eos_token, int max_draft_tokens) {
  CoreConfig c;
  c.num_pages = num_pages;
  c.num_host_pages = num_host_pages;
  c.max_seqs = max_seqs;
  c.max_tokens_per_step = max_tokens_per_step;
  c.max_pages_per_seq = max_pages_per_seq;
  c.prefill_chunk = prefill_chunk;
  c.token_multiple = token_multiple;
  c.policy = static_cast<Policy>(policy);
  c.preempt = static_cast<PreemptMode>(preempt_mode);
  c.enable_prefix_cache = enable_prefix_cache != 0;
  c.eos_token = eos_token;
  c.max_draft_tokens = max_draft_tokens;
  return new Core(c);
}
void ogb_core_destroy(void* h) { delete static_cast<Core*>(h); }
void ogb_core_set_window(void* h, int window, int sink_tokens) { static_cast<Core*>(h)->set_window(window, sink_tokens); }
int ogb_core_released_pages(void* h, int64_t seq_id) { return static_cast<Core*>(h)->released_pages(seq_id); }
int ogb_core_layout(void* h, int32_t* out, int cap) {
  const PlanLayout& l = static_cast<Core*>(h)->layout();
  const int32_t v[] = {l.header, l.token_ids, l.positions, l.slots, l.seq_slot, l.ctx_len, l.cu_q, l.page_table,
                       l.tile_seq, l.tile_q0, l.logit_rows, l.temperature, l.top_k, l.top_p, l.min_p, l.uniform,
                       l.copy_src, l.copy_dst, l.swap_out_dev, l.swap_out_host, l.swap_in_dev, l.swap_in_host,
                       l.total_words, l.max_tiles, l.max_swap, l.logit_seq, l.max_rows, l.move_runs, l.max_runs};
  const int n = static_cast<int>(sizeof(v) / sizeof(v[0]));
  for (int i = 0; i < n && i < cap; ++i) out[i] = v[i];
  return n;
}
int64_t ogb_core_add_request(void* h, const int32_t* prompt, int n, int max_new_tokens, float temperature, int top_k,
                             float top_p, float min_p, uint64_t seed, int priority, int tenant, int ignore_eos,
                             const int32_t* stop_ids, int n_stop) {
  SamplingParams sp;
  sp.temperature = temperature;
  sp.top_k = top_k;
  sp.top_p = top_p;
  sp.min_p = min_p;
  sp.seed = seed;
  return static_cast<Core*>(h)->add_request(prompt, n, max_new_tokens, sp, priority, tenant, ignore_eos != 0, stop_ids, n_stop);
}
int ogb_core_build_step(void* h, int32_t* plan) { return static_cast<Core*>(h)->build_step(plan); }
int ogb_core_commit_step(void* h, const int32_t* sampled, int n, int64_t* ev_seq, int32_t* ev_token, int32_t* ev_finish,
                         int max_events) {
  std::vector<StepEvent> ev(max_events > 0 ? max_events : 1);
  const int ne = static_cast<Core*>(h)->commit_step(sampled, n, ev.data(), max_events);
  for (int i = 0; i < ne; ++i) { ev_seq[i] = ev[i].seq_id; ev_token[i] = ev[i].token; ev_finish[i] = ev[i].finish; }
  return ne;
}
int ogb_core_cancel(void* h, int64_t id) { return static_cast<Core*>(h)->cancel(id) ? 1 : 0; }
int64_t ogb_core_fork(void* h, int64_t id) { return static_cast<Core*>(h)->fork(id); }
int ogb_core_swap_state(void* h, int64_t a, int64_t b) { return static_cast<Core*>(h)->swap_state(a, b) ? 1 : 0; }
int ogb_core_rewind(void* h, int64_t id, int new_len) { return static_cast<Core*>(h)->rewind(id, new_len) ? 1 : 0; }
int ogb_core_set_draft(void* h, int64_t id, const int32_t* tokens, int k) {
  return static_cast<Core*>(h)->set_draft(id, tokens, k) ? 1 : 0;
}
int ogb_core_append_tokens(void* h, int64_t id, const int32_t* tokens, int n) {
  return static_cast<Core*>(h)->append_tokens(id, tokens, n) ? 1 : 0;
}
int ogb_core_seq_pages(void* h, int64_t id, int32_t* out, int cap) { return static_cast<Core*>(h)->seq_pages(id, out, cap); }
int ogb_core_prefix_adopt(void* h, const int32_t* tokens, int n, int32_t* out_pages, int cap) {
  return static_cast<Core*>(h)->prefix_adopt(tokens, n, out_pages, cap);
}
int ogb_core_prefix_unpublish(void* h, const int32_t* pages, int n) { return static_cast<Core*>(h)->prefix_unpublish(pages, n); }
int ogb_core_prefix_peek(void* h, const int32_t* tokens, int n, int32_t* out_pages, int cap) {
  return static_cast<Core*>(h)->prefix_peek(tokens, n, out_pages, cap);
}
int ogb_core_seq_len(void* h, int64_t id) { return static_cast<Core*>(h)->seq_len(id); }
int ogb_core_seq_computed(void* h, int64_t id) { return static_cast<Core*>(h)->seq_computed(id); }
int ogb_core_seq_tokens(void* h, int64_t id, int32_t* out, int cap) { return static_cast<Core*>(h)->seq_tokens(id, out, cap); }
void ogb_core_release(void* h, int64_t id) { static_cast<Core*>(h)->release(id); }
void ogb_core_add_pages(void* h, int n) { static_cast<Core*>(h)->add_pages(n); }
int64_t ogb_core_stat(void* h, int which) {
  Core* c = static_cast<Core*>(h);
  switch (which) {
    case 0: return c->num_waiting();
    case 1: return c->num_running();
    case 2: return c->num_swapped();
    case 3: return c->num_free_pages();
    case 4: return c->prefix_hits();
    case 5: return c->prefix_lookups();
    case 6: return c->num_preemptions();
    case 7: return c->has_work() ? 1 : 0;
    case 8: return c->spec_proposed();
    case 9: return c->spec_accepted();
    case 10: return c->spec_steps();
    case 11: return c->num_pages();
    default: return -1;
  }
}

}  // extern "C"

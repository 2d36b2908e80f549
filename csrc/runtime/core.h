// Host runtime core: paged-KV block pool, prefix cache, continuous-batching scheduler and the
// step builder that fills one packed int32 plan per engine step.
//
// What it covers of the reference:
//   * page table / pages / CoW fork / rewind / checkpoint (crates/onnx-genai-kv/src/page_table.rs:943-1905,
//     paged_cache.rs:913-1085) -- here page *ids* only; the bytes live in the device pool that the
//     attention kernels read directly;
//   * prefix radix trie with ref-counted pages (crates/onnx-genai-kv/src/prefix_cache.rs:24-370) -- here
//     a chained block hash -> page map with LRU reuse of unreferenced cached pages;
//   * scheduler: FCFS / priority / fair-share admission, token and page budgets, swap or recompute
//     preemption (crates/onnx-genai-scheduler/src/lib.rs:133-145,245-601, policy.rs:7-80);
//   * continuous batching (crates/onnx-genai-engine/src/batched.rs:340-368,663-749) -- but with chunked
//     multi-token prefill mixed into decode steps and preemption of batched rows, which the
//     reference's one-token-per-row manager does not do;
//   * per-request RNG: one uniform per sampled token, independent of the batch row
//     (crates/onnx-genai-engine/src/sampling.rs:9-32).
#pragma once
#include <cstdint>
#include <deque>
#include <string>
#include <unordered_map>
#include <vector>

namespace ogb {

constexpr int kPageTokens = 16;

enum class SeqStatus : int { Waiting = 0, Running = 1, Swapped = 2, Finished = 3 };
enum class FinishReason : int { None = 0, Length = 1, Stop = 2, Cancelled = 3, Error = 4 };
enum class Policy : int { Fcfs = 0, Priority = 1, FairShare = 2 };
enum class PreemptMode : int { Recompute = 0, Swap = 1 };

struct SamplingParams {
  float temperature = 0.f;  // <= 0: greedy
  int top_k = 0;
  float top_p = 1.f;
  float min_p = 0.f;
  uint64_t seed = 0;
};

struct Sequence {
  int64_t id = 0;
  std::vector<int32_t> tokens;   // prompt + generated
  int prompt_len = 0;
  int num_computed = 0;          // tokens whose K/V are in the cache
  int max_new_tokens = 0;
  int priority = 0;              // higher runs first under Policy::Priority
  int tenant = 0;                // fair-share bucket
  int64_t arrival = 0;
  bool ignore_eos = false;
  std::vector<int32_t> stop_ids;
  SamplingParams sampling;
  uint64_t rng_state = 0;
  SeqStatus status = SeqStatus::Waiting;
  FinishReason finish = FinishReason::None;
  std::vector<int32_t> pages;        // device page ids, one per 16 tokens; -1 = released (see Core::set_window)
  int trim_end = 0;                  // pages [sink pages, trim_end) have been released under the sliding window
  std::vector<int32_t> host_pages;   // swap space page ids while Swapped
  int num_cached_prefix = 0;         // tokens served from the prefix cache at admission
  int scheduled = 0;                 // tokens scheduled in the step being built
  bool samples_this_step = false;
  int num_draft = 0;                 // speculative tokens appended to `tokens` for the step being built
  std::vector<int32_t> draft;        // proposed continuation waiting to be verified
};

// Reference-counted device pages with a prefix cache over full pages.
class BlockPool {
 public:
  explicit BlockPool(int num_pages);
  int num_pages() const { return static_cast<int>(ref_.size()); }
  int num_free() const { return static_cast<int>(free_.size()) + evictable_live_; }
  int allocate();                    // -1 when exhausted
  void add_pages(int n);             // the backing buffer grew: ids [old size, old size + n) become free pages
  void retain(int page) { ++ref_[page]; }
  void release(int page);            // refcount--; cached pages become evictable, others free
  int refcount(int page) const { return ref_[page]; }
  // prefix cache
  static uint64_t chain_hash(uint64_t parent, const int32_t* tokens, int n);
  int lookup(uint64_t hash);         // page id (retained) or -1
  bool contains(uint64_t hash) const { return by_hash_.count(hash) != 0; }
  int peek(uint64_t hash) const { auto it = by_hash_.find(hash); return it == by_hash_.end() ? -1 : it->second; }
  void publish(int page, uint64_t hash);
  bool unpublish(int page);          // a cached, unreferenced page leaves the prefix cache and becomes free again
  int64_t hits() const { return hits_; }
  int64_t lookups() const { return lookups_; }
  void reset_prefix_cache();

 private:
  std::vector<int> ref_;
  std::vector<uint64_t> hash_of_;    // 0 = not cached
  std::vector<int> free_;
  std::deque<int> evictable_;        // cached, refcount 0, LRU order (front = oldest)
  std::vector<uint8_t> in_evictable_;
  int evictable_live_ = 0;           // deque entries that are live (the deque also holds stale ones, skipped lazily)
  std::unordered_map<uint64_t, int> by_hash_;
  int64_t hits_ = 0, lookups_ = 0;
};

struct CoreConfig {
  int num_pages = 0;
  int num_host_pages = 0;        // swap space
  int max_seqs = 256;            // concurrent running sequences
  int max_tokens_per_step = 2048;
  int max_pages_per_seq = 256;
  int prefill_chunk = 2048;      // per-sequence cap of prompt tokens per step
  int token_multiple = 1;        // pad-free rounding of the step size (prefill chunks shrink to fit)
  Policy policy = Policy::Fcfs;
  PreemptMode preempt = PreemptMode::Recompute;
  bool enable_prefix_cache = true;
  int eos_token = -1;
  int max_draft_tokens = 0;      // speculative decoding: draft tokens verified per sequence per step
};

// Offsets (in int32 words) of the sections of a packed step plan.
struct PlanLayout {
  int header = 0;        // 32 words
  int token_ids, positions, slots;           // [max_tokens]
  int seq_slot, ctx_len;                     // [max_seqs]
  int cu_q;                                  // [max_seqs + 1]  (prefill rows only, relative to first prefill token)
  int page_table;                            // [max_seqs * max_pages_per_seq]
  int tile_seq, tile_q0;                     // [max_tiles]
  int logit_rows;                            // [max_seqs]
  int temperature, top_k, top_p, min_p, uniform;  // [max_rows] (floats stored by bit pattern)
  int logit_seq;                             // [max_rows] sequence id (low 31 bits) of every logit row
  int copy_src, copy_dst;                    // [max_seqs] CoW page copies to run before the step
  int swap_out_dev, swap_out_host, swap_in_dev, swap_in_host;  // [max_swap]
  int move_runs;                             // [2 * max_runs] (kind, count) pairs: the order in which the page moves above were
                                             // decided (kind 0 = CoW copy, 1 = swap out, 2 = swap in); each list is consumed
                                             // front to back, so running the runs in order reproduces the scheduler's sequence
  int total_words;
  int max_tiles, max_swap, max_runs;
  int max_rows;                              // max_seqs * (1 + max_draft_tokens)
};

enum PlanHeader : int {
  kHdrNumTokens = 0, kHdrNumDecode, kHdrNumPrefillSeqs, kHdrNumTiles, kHdrNumLogitRows, kHdrNumCopies,
  kHdrNumSwapOut, kHdrNumSwapIn, kHdrNumPrefillTokens, kHdrMaxCtx, kHdrNumPreempted, kHdrStepId, kHdrNumMoveRuns,
};

struct StepEvent {
  int64_t seq_id;
  int32_t token;      // -1 when the event only reports a state change
  int32_t finish;     // FinishReason
};

class Core {
 public:
  explicit Core(const CoreConfig& cfg);
  const CoreConfig& config() const { return cfg_; }
  const PlanLayout& layout() const { return layout_; }

  int64_t add_request(const int32_t* prompt, int n, int max_new_tokens, const SamplingParams& sp, int priority, int tenant,
                      bool ignore_eos, const int32_t* stop_ids, int n_stop);
  bool cancel(int64_t seq_id);
  // Builds the next step into `plan` (layout().total_words int32 words).  Returns the number of tokens scheduled.
  int build_step(int32_t* plan);
  // Consumes the sampled tokens of the last built step (one per logit row, in row order).
  int commit_step(const int32_t* sampled, int n, StepEvent* events, int max_events);

  // session-style operations on a live sequence
  int64_t fork(int64_t seq_id);                    // copy-on-write clone (shares pages)
  // The two sequences exchange everything but their ids and arrival order (tokens, pages, progress, status); used between
  // steps when a forked branch of a speculation tree won and the caller's id has to continue as that branch.
  bool swap_state(int64_t a, int64_t b);
  bool rewind(int64_t seq_id, int new_len);
  // Sliding-window retention with attention sinks (the policy of crates/onnx-genai-kv/src/paged_cache.rs:483-585, kept
  // position-indexed instead of compacted): once a sequence has run `window` + slack tokens past a page, no later query
  // can see it, so every page that lies wholly between the first ceil(sink_tokens / 16) pages and the window is released
  // and its page-table entry becomes -1 (the attention kernels never read those entries).  window <= 0 turns it off.
  // A rewind that would bring released keys back into view is refused.
  void set_window(int window, int sink_tokens);
  int released_pages(int64_t seq_id) const;        // drop trailing tokens and their pages
  int seq_len(int64_t seq_id) const;
  int seq_computed(int64_t seq_id) const;          // tokens whose K/V are in the cache, -1 for an unknown id
  int seq_tokens(int64_t seq_id, int32_t* out, int cap) const;
  // Speculative decoding: propose `k` tokens to follow the sequence's last token.  The next step feeds the
  // last token plus the drafts, samples every position, and commit_step keeps the longest prefix of the
  // drafts that the samples confirm (plus the correction / bonus token), rewinding the KV pages of the rest.
  bool set_draft(int64_t seq_id, const int32_t* tokens, int k);
  // Extends a live sequence with tokens chosen by the caller (they count as prompt: the next steps compute
  // their K/V as a prefill chunk and sample after the last one).  With rewind this lets a caller re-align a
  // sequence to a corrected continuation without re-submitting the prefix.
  bool append_tokens(int64_t seq_id, const int32_t* tokens, int n);
  // KV offload connector support.  seq_pages: the device pages of a live sequence that hold computed tokens.
  // prefix_adopt: for every full page of `tokens` that the prefix cache does not serve yet, allocate a page and
  // register it under the page's chained hash as a cached, unreferenced page; the caller then fills those pages
  // with K/V fetched from outside the device.  out_pages[i] = adopted page id, or -1 where a page already
  // existed; returns the number of leading pages that are now served (stops when the pool is exhausted).
  int seq_pages(int64_t seq_id, int32_t* out, int cap) const;
  int prefix_adopt(const int32_t* tokens, int n_tokens, int32_t* out_pages, int cap);
  // prefix_unpublish: adopted pages that were never filled (the pool ran out in the middle of a chunk) leave the
  // prefix cache again, so no later request can attach to uninitialised K/V.  Returns how many were removed.
  int prefix_unpublish(const int32_t* pages, int n);
  // prefix_peek: the pages that currently serve the leading full pages of `tokens` (no reference is taken; valid
  // until the next call that allocates).  Returns how many leading pages are cached.
  int prefix_peek(const int32_t* tokens, int n_tokens, int32_t* out_pages, int cap) const;
  int64_t spec_proposed() const { return spec_proposed_; }
  int64_t spec_accepted() const { return spec_accepted_; }
  int64_t spec_steps() const { return spec_steps_; }
  void release(int64_t seq_id);                    // forget a finished sequence

  int num_waiting() const { return static_cast<int>(waiting_.size()); }
  int num_running() const { return static_cast<int>(running_.size()); }
  int num_swapped() const { return static_cast<int>(swapped_.size()); }
  int num_free_pages() const { return pool_.num_free(); }
  int num_pages() const { return pool_.num_pages(); }
  void add_pages(int n) { pool_.add_pages(n); cfg_.num_pages = pool_.num_pages(); }   // KV buffers grow in place
  int64_t prefix_hits() const { return pool_.hits(); }
  int64_t prefix_lookups() const { return pool_.lookups(); }
  int64_t num_preemptions() const { return preemptions_; }
  bool has_work() const { return !waiting_.empty() || !running_.empty() || !swapped_.empty(); }

 private:
  Sequence* find(int64_t id);
  const Sequence* find(int64_t id) const;
  bool ensure_pages(Sequence& s, int new_len, std::vector<std::pair<int, int>>& copies);
  void free_pages(Sequence& s, bool publish_prefix);
  void trim_window(Sequence& s);
  void try_prefix_attach(Sequence& s);
  void publish_full_pages(Sequence& s);
  bool preempt_one(Sequence* keep, std::vector<std::pair<int, int>>& swap_out);
  std::vector<int64_t> waiting_order();
  float next_uniform(Sequence& s);
  void finish(Sequence& s, FinishReason why);

  CoreConfig cfg_;
  PlanLayout layout_;
  BlockPool pool_;
  std::vector<int> host_free_;
  std::unordered_map<int64_t, Sequence> seqs_;
  std::deque<int64_t> waiting_;
  std::vector<int64_t> running_;
  std::deque<int64_t> swapped_;
  std::vector<int64_t> step_rows_;       // sequence of each logit row of the last built step
  std::vector<int64_t> step_seqs_;       // every sequence scheduled in the last built step
  std::vector<uint8_t> move_kinds_;      // kind of every page move of the step being built, in decision order
  std::unordered_map<int, int64_t> tenant_served_;
  int64_t next_id_ = 1;
  int64_t clock_ = 0;
  int64_t step_id_ = 0;
  int64_t preemptions_ = 0;
  int window_ = 0, sink_pages_ = 0;   // sliding-window retention (set_window)
  int64_t spec_proposed_ = 0, spec_accepted_ = 0, spec_steps_ = 0;
};

}  // namespace ogb

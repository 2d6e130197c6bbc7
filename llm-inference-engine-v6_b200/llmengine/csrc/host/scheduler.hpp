// Continuous-batching scheduler: the decisions only. It never touches the device; the caller runs
// the planned batch through the step function and hands the sampled tokens back.
//
//   plan()   -> finalize finished requests (pages and slot go back), admit waiting ones, choose
//               this step's batch, reserve its pages
//   commit() -> take the sampled token of every wanted row, advance cursors, finish requests
//
// State machine, knobs and finish reasons are the reference's ContinuousBatchScheduler
// (src/scheduler.cpp:136-319; include/llmengine/scheduler.hpp:92-147): WAITING -> PREFILLING ->
// RUNNING -> FINISHED; FIFO admission while running+prefilling < max_concurrent (no look at free
// pages); one prefill-token budget per step shared first-come first-served, decode tokens not
// counted; "stop" (EOS, not appended), "length", "capacity". Differences: a step is ONE mixed batch
// (prompt portions beside one token per running request) instead of the reference's two phases, so
// a request whose prompt ends in step k decodes from step k+1 (token streams are the same); and
// pages are reserved before the step rather than discovered missing inside it. When pages run out
// the request that could not reserve ends with "capacity" and keeps what it generated; nothing is
// preempted, recomputed or made to wait (src/scheduler.cpp:190-194,266-270).
#pragma once

#include "cache_manager.hpp"

#include <deque>
#include <memory>
#include <set>
#include <string>

namespace llmhost {

enum class SeqState { WAITING, PREFILLING, RUNNING, FINISHED };

struct SequenceResult {
  std::int64_t seq_id = 0;
  int prompt_len = 0;
  std::vector<std::int32_t> token_ids;  // prompt + generated
  std::string finish_reason;            // "stop" | "length" | "capacity" | "error"
};

struct Sequence {
  std::int64_t seq_id = 0;
  std::vector<std::int32_t> token_ids;
  int prompt_len = 0;
  int cursor = 0;  // tokens already run through the model
  int max_new_tokens = 0;
  float temperature = 0.f;
  std::int32_t seed = 0;
  SeqState state = SeqState::WAITING;
  std::string finish_reason;
  int step_tokens = 0;       // tokens of this request in the planned step
  bool step_samples = false;  // the planned step yields a token for it
};

class Scheduler {
 public:
  Scheduler(CacheManager& cm, int vocab_size, int max_positions, std::set<int> eos_token_ids,
            int max_concurrent = 64, int max_prefill_tokens_per_step = 256, std::int64_t id_base = 0,
            int portion_multiple = 1);

  std::int64_t enqueue(std::vector<std::int32_t> prompt, int max_new_tokens, float temperature = 0.f,
                       std::int32_t seed = 0);

  // The next step's batch (empty when there is nothing to run). Must be followed by commit()
  // with one token per wanted row, in the order of the entries, before the next plan().
  const std::vector<StepEntry>& plan();
  void commit(const std::vector<std::int32_t>& sampled);
  // The planned step could not be run (the device reported a failure): its requests end with
  // `reason` ("error", as the reference's streaming path names it, include/llmengine/engine.hpp:90),
  // keep what they had generated, and give their pages back at the next plan(). Requests that were
  // not part of the step go on.
  void fail_step(const std::string& reason);
  // Finalizes what is finished without planning (the end of run_until_idle in the reference).
  void finalize();

  bool idle() const { return waiting_.empty() && prefilling_.empty() && running_.empty(); }
  bool has_unfinished() const;
  bool plan_open() const { return plan_open_; }  // a planned step awaits commit() or fail_step()
  std::vector<SequenceResult> results() const;  // sorted by seq_id
  void clear_results() { results_.clear(); }
  int budget() const { return budget_; }
  void set_budget(int b);
  int max_concurrent() const { return max_concurrent_; }
  // A prompt portion that is not the prompt's last ends at a position that is a multiple of this
  // (1: anywhere). Mixers whose state can only be carried over at such points ask for it.
  int portion_multiple() const { return portion_multiple_; }
  int num_waiting() const { return static_cast<int>(waiting_.size()); }
  int num_prefilling() const { return static_cast<int>(prefilling_.size()); }
  int num_running() const { return static_cast<int>(running_.size()); }
  // Cache-manager ids of the requests admitted by the last plan() (their state slots are fresh).
  const std::vector<std::int64_t>& last_admitted() const { return last_admitted_; }
  // Requests are known to the cache manager as id_base + seq_id, so that several schedulers can
  // share one manager.
  std::int64_t cache_id(const Sequence& s) const { return id_base_ + s.seq_id; }

 private:
  void finalize_list(std::vector<std::unique_ptr<Sequence>>& list);
  void finish(Sequence& s, const char* reason);
  void take_token(Sequence& s, std::int32_t token);

  CacheManager& cm_;
  int vocab_size_, max_positions_;
  std::set<int> eos_;
  int max_concurrent_, budget_, portion_multiple_;
  std::int64_t id_base_ = 0;
  std::int64_t next_id_ = 0;
  std::vector<std::int64_t> last_admitted_;
  std::deque<std::unique_ptr<Sequence>> waiting_;
  std::vector<std::unique_ptr<Sequence>> prefilling_, running_;
  std::vector<SequenceResult> results_;
  std::vector<StepEntry> plan_;
  std::vector<Sequence*> plan_seqs_;
  bool plan_open_ = false;
};

}  // namespace llmhost

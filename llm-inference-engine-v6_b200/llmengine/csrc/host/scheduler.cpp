#include "scheduler.hpp"

#include <algorithm>
#include <stdexcept>

namespace llmhost {

Scheduler::Scheduler(CacheManager& cm, int vocab_size, int max_positions, std::set<int> eos_token_ids,
                     int max_concurrent, int max_prefill_tokens_per_step, std::int64_t id_base, int portion_multiple)
    : cm_(cm), vocab_size_(vocab_size), max_positions_(max_positions), eos_(std::move(eos_token_ids)),
      max_concurrent_(max_concurrent), budget_(max_prefill_tokens_per_step), portion_multiple_(portion_multiple),
      id_base_(id_base) {
  // Same guards as the reference (src/scheduler.cpp:143-150): without them the loop never ends.
  if (max_concurrent_ <= 0) throw std::invalid_argument("ContinuousBatchScheduler: max_concurrent must be >= 1");
  if (budget_ <= 0) throw std::invalid_argument("ContinuousBatchScheduler: max_prefill_tokens_per_step must be >= 1");
  if (vocab_size_ <= 0 || max_positions_ <= 0) throw std::invalid_argument("ContinuousBatchScheduler: bad model sizes");
  if (portion_multiple_ <= 0) throw std::invalid_argument("ContinuousBatchScheduler: portion_multiple must be >= 1");
  // a budget below the multiple could never cut a long prompt: the loop would not end
  if (budget_ < portion_multiple_)
    throw std::invalid_argument("ContinuousBatchScheduler: max_prefill_tokens_per_step must be at least the model's portion multiple " +
                                std::to_string(portion_multiple_));
}

void Scheduler::set_budget(int b) {
  if (b <= 0) throw std::invalid_argument("ContinuousBatchScheduler: max_prefill_tokens_per_step must be >= 1");
  if (b < portion_multiple_)
    throw std::invalid_argument("ContinuousBatchScheduler: max_prefill_tokens_per_step must be at least the model's portion multiple " +
                                std::to_string(portion_multiple_));
  budget_ = b;
}

std::int64_t Scheduler::enqueue(std::vector<std::int32_t> prompt, int max_new_tokens, float temperature,
                                std::int32_t seed) {
  // Input contract of the reference's enqueue (src/scheduler.cpp:153-175).
  if (prompt.empty()) throw std::invalid_argument("enqueue: prompt is empty");
  if (max_new_tokens < 0) throw std::invalid_argument("enqueue: max_new_tokens negative");
  if (!(temperature >= 0.f)) throw std::invalid_argument("enqueue: temperature must be >= 0");
  for (auto t : prompt)
    if (t < 0 || t >= vocab_size_)
      throw std::invalid_argument("enqueue: token id " + std::to_string(t) + " out of range [0, " +
                                  std::to_string(vocab_size_) + ")");
  if (static_cast<std::int64_t>(prompt.size()) + max_new_tokens > max_positions_)
    throw std::invalid_argument("enqueue: prompt + max_new_tokens exceeds the position limit " +
                                std::to_string(max_positions_));
  auto s = std::make_unique<Sequence>();
  s->seq_id = next_id_++;
  s->prompt_len = static_cast<int>(prompt.size());
  s->token_ids = std::move(prompt);
  s->max_new_tokens = max_new_tokens;
  s->temperature = temperature;
  s->seed = seed;
  const std::int64_t id = s->seq_id;
  waiting_.push_back(std::move(s));
  return id;
}

void Scheduler::finish(Sequence& s, const char* reason) {
  s.state = SeqState::FINISHED;
  s.finish_reason = reason;
}

void Scheduler::finalize_list(std::vector<std::unique_ptr<Sequence>>& list) {
  std::vector<std::unique_ptr<Sequence>> keep;
  for (auto& s : list) {
    if (s->state != SeqState::FINISHED) {
      keep.push_back(std::move(s));
      continue;
    }
    if (cm_.has_request(cache_id(*s))) cm_.release(cache_id(*s));
    SequenceResult r;
    r.seq_id = s->seq_id;
    r.prompt_len = s->prompt_len;
    r.token_ids = s->token_ids;
    r.finish_reason = s->finish_reason;
    results_.push_back(std::move(r));
  }
  list.swap(keep);
}

void Scheduler::finalize() {
  if (plan_open_) throw std::logic_error("finalize: a planned step has not been committed");
  finalize_list(prefilling_);
  finalize_list(running_);
}

bool Scheduler::has_unfinished() const {
  if (!waiting_.empty()) return true;
  for (const auto& s : prefilling_) if (s->state != SeqState::FINISHED) return true;
  for (const auto& s : running_) if (s->state != SeqState::FINISHED) return true;
  return false;
}

const std::vector<StepEntry>& Scheduler::plan() {
  if (plan_open_) throw std::logic_error("plan: the previous step has not been committed");
  finalize_list(prefilling_);
  finalize_list(running_);

  last_admitted_.clear();
  while (!waiting_.empty() && static_cast<int>(running_.size() + prefilling_.size()) < max_concurrent_) {
    const int slot = cm_.add_request(cache_id(*waiting_.front()));
    if (slot < 0) break;  // no state slot free: wait for a request to finish
    last_admitted_.push_back(cache_id(*waiting_.front()));
    auto s = std::move(waiting_.front());
    waiting_.pop_front();
    s->state = SeqState::PREFILLING;
    prefilling_.push_back(std::move(s));
  }

  plan_.clear();
  plan_seqs_.clear();
  int budget = budget_;
  for (auto& sp : prefilling_) {
    Sequence& s = *sp;
    s.step_tokens = 0;
    s.step_samples = false;
    if (s.state == SeqState::FINISHED || budget <= 0) continue;
    int n = std::min(s.prompt_len - s.cursor, budget);
    // a portion that leaves some of the prompt for later ends at a multiple of portion_multiple_
    if (n < s.prompt_len - s.cursor && portion_multiple_ > 1) n = (s.cursor + n) / portion_multiple_ * portion_multiple_ - s.cursor;
    if (n <= 0) continue;
    if (!cm_.reserve(cache_id(s), n)) {
      finish(s, "capacity");
      continue;
    }
    StepEntry e;
    e.id = cache_id(s);
    e.tokens.assign(s.token_ids.begin() + s.cursor, s.token_ids.begin() + s.cursor + n);
    if (s.cursor + n == s.prompt_len && s.max_new_tokens > 0) {
      e.want.push_back(n - 1);
      s.step_samples = true;
    }
    e.temperature = s.temperature;
    e.seed = s.seed;
    e.draw = 0;
    s.step_tokens = n;
    budget -= n;
    plan_.push_back(std::move(e));
    plan_seqs_.push_back(&s);
  }
  for (auto& sp : running_) {
    Sequence& s = *sp;
    s.step_tokens = 0;
    s.step_samples = false;
    if (s.state == SeqState::FINISHED) continue;
    if (!cm_.reserve(cache_id(s), 1)) {
      finish(s, "capacity");
      continue;
    }
    StepEntry e;
    e.id = cache_id(s);
    e.tokens.push_back(s.token_ids.back());
    e.want.push_back(0);
    e.temperature = s.temperature;
    e.seed = s.seed;
    e.draw = static_cast<std::int32_t>(s.token_ids.size()) - s.prompt_len;
    s.step_tokens = 1;
    s.step_samples = true;
    plan_.push_back(std::move(e));
    plan_seqs_.push_back(&s);
  }
  plan_open_ = !plan_.empty();
  return plan_;
}

void Scheduler::take_token(Sequence& s, std::int32_t token) {
  // src/scheduler.cpp:207-227 and 271-281: EOS ends without being appended; the cap is checked
  // right after the push so max_new_tokens = 1 yields exactly one token.
  if (token < 0 || token >= vocab_size_) throw std::invalid_argument("commit: sampled token out of range");
  if (eos_.count(token)) {
    finish(s, "stop");
    return;
  }
  s.token_ids.push_back(token);
  if (static_cast<int>(s.token_ids.size()) - s.prompt_len >= s.max_new_tokens) {
    finish(s, "length");
    return;
  }
  s.state = SeqState::RUNNING;
}

void Scheduler::commit(const std::vector<std::int32_t>& sampled) {
  if (!plan_open_) throw std::logic_error("commit: no planned step");
  std::size_t want = 0;
  for (Sequence* s : plan_seqs_) want += s->step_samples ? 1 : 0;
  if (sampled.size() != want)
    throw std::invalid_argument("commit: expected " + std::to_string(want) + " sampled tokens, got " +
                                std::to_string(sampled.size()));
  std::size_t r = 0;
  for (Sequence* sp : plan_seqs_) {
    Sequence& s = *sp;
    cm_.advance(cache_id(s), s.step_tokens);
    s.cursor += s.step_tokens;
    if (s.step_samples) {
      take_token(s, sampled[r++]);
    } else if (s.state == SeqState::PREFILLING && s.cursor == s.prompt_len) {
      finish(s, "length");  // max_new_tokens == 0: nothing is sampled (src/scheduler.cpp:201-206)
    }
  }
  // requests whose prompt ended move to the running list, in order
  std::vector<std::unique_ptr<Sequence>> still;
  for (auto& s : prefilling_) {
    if (s->state == SeqState::RUNNING) running_.push_back(std::move(s));
    else still.push_back(std::move(s));
  }
  prefilling_.swap(still);
  plan_.clear();
  plan_seqs_.clear();
  plan_open_ = false;
}

void Scheduler::fail_step(const std::string& reason) {
  if (!plan_open_) throw std::logic_error("fail_step: no planned step");
  for (Sequence* s : plan_seqs_) {
    s->step_tokens = 0;
    s->step_samples = false;
    finish(*s, reason.c_str());
  }
  plan_.clear();
  plan_seqs_.clear();
  plan_open_ = false;
}

std::vector<SequenceResult> Scheduler::results() const {
  std::vector<SequenceResult> out = results_;
  std::sort(out.begin(), out.end(), [](const SequenceResult& a, const SequenceResult& b) { return a.seq_id < b.seq_id; });
  return out;
}

}  // namespace llmhost

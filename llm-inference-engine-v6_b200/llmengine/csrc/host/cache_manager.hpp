// Host-side bookkeeping of the paged cache: which pages and which state slot each live request
// holds. It owns no device memory; page ids index the page tensors that the engine allocates.
//
// The reference keeps one pool for all layers (BlockManager, src/paged_kv.cpp:8-66: FIFO free list,
// allocate pops the front, free pushes to the back) and one block table per sequence
// (PagedKVCache, src/paged_kv.cpp:70-139: entry i covers positions [i*bs, (i+1)*bs), grown one block
// at a time inside write). Here:
//   * layers are put into groups by what they must keep (all keys, or a window of the last W);
//     every group has its own pool and every request one block table per group;
//   * pages are reserved before a step for all tokens the step brings (all groups or none), so a
//     step can never fail half-way;
//   * a window group gives a page back as soon as no later query can see any of its positions;
//   * every request also holds one state slot (fixed-size per-request state of mixers that have
//     some; this architecture has none, the slot is still handed out and taken back).
#pragma once

#include <cstdint>
#include <deque>
#include <map>
#include <string>
#include <unordered_map>
#include <vector>

namespace llmhost {

struct GroupSpec {
  int num_pages = 0;
  int window = 0;  // 0: keep every key; W > 0: a query at position p reads keys p-W+1 .. p
};

class CacheManager {
 public:
  CacheManager(int page_size, std::vector<GroupSpec> groups, int num_slots);

  int page_size() const { return page_size_; }
  int num_groups() const { return static_cast<int>(groups_.size()); }
  int num_pages(int g) const { return group(g).spec.num_pages; }
  int window(int g) const { return group(g).spec.window; }
  int free_pages(int g) const { return static_cast<int>(group(g).free_list.size()); }
  int num_slots() const { return num_slots_; }
  int free_slots() const { return static_cast<int>(free_slots_.size()); }
  int num_requests() const { return static_cast<int>(requests_.size()); }

  // Registers a request and gives it a state slot. Returns the slot, or -1 if none is free.
  int add_request(std::int64_t id);
  bool has_request(std::int64_t id) const { return requests_.count(id) != 0; }
  int length(std::int64_t id) const { return req(id).length; }
  int reserved(std::int64_t id) const { return req(id).reserved; }
  int slot(std::int64_t id) const { return req(id).slot; }

  // Pages for positions [length, length + n_new) in every group, all or nothing.
  bool reserve(std::int64_t id, int n_new);
  // The step that brought n tokens is on its way: length += n; pages a window has passed go back.
  void advance(std::int64_t id, int n);
  // Everything the request holds goes back (pages of every group, the slot).
  void release(std::int64_t id);

  // Entry i covers positions [i*page_size, (i+1)*page_size); -1 once the page has been given back.
  const std::vector<int>& block_table(std::int64_t id, int g) const;
  std::vector<std::int64_t> request_ids() const;

  // Throws std::logic_error naming the first broken invariant: every page is either free or held
  // by exactly one request, never both, never twice; same for slots; tables cover the lengths.
  void check() const;

 private:
  struct Group {
    GroupSpec spec;
    std::deque<int> free_list;
  };
  struct Request {
    int slot = -1;
    int length = 0;    // tokens whose keys are in the cache (or on their way)
    int reserved = 0;  // positions [0, reserved) are covered by pages (where still needed)
    std::vector<std::vector<int>> tables;  // per group
  };
  const Group& group(int g) const;
  const Request& req(std::int64_t id) const;
  Request& req(std::int64_t id);
  int pages_for(int tokens) const { return (tokens + page_size_ - 1) / page_size_; }

  int page_size_;
  int num_slots_;
  std::vector<Group> groups_;
  std::deque<int> free_slots_;
  std::map<std::int64_t, Request> requests_;
};

// ------------------------------------------------------------------------------------------------
// One step's batch: for each request its next tokens and the places among them whose logits are
// wanted. Prompt portions of any length stand beside single decoded tokens.
struct StepEntry {
  std::int64_t id = 0;
  std::vector<std::int32_t> tokens;
  std::vector<std::int32_t> want;  // indices into tokens
  // sampling parameters of the wanted rows (used by the scheduler's steps only)
  float temperature = 0.f;
  std::int32_t seed = 0;
  std::int32_t draw = 0;
};

// Where each array of a step lies in the int32 staging buffer (element offsets), for capacities
// chosen by the caller. The same layout is used on the host (pinned) and on the device.
struct StepLayout {
  int cap_tokens = 0, cap_seqs = 0, cap_rows = 0, max_blocks = 0, num_groups = 0;
  int token_ids = 0, positions = 0, token_seq = 0, logit_rows = 0;
  int row_temperature = 0, row_seed = 0, row_draw = 0;  // temperature: float bits
  int seq_start = 0, seq_ntok = 0, seq_qoff = 0, seq_slot = 0, seq_len = 0;
  int block_tables = 0;  // [num_groups][cap_seqs][max_blocks]
  int total = 0;         // elements
  static StepLayout make(int cap_tokens, int cap_seqs, int cap_rows, int max_blocks, int num_groups);
};

struct StepCounts {
  int n_tokens = 0, n_seqs = 0, n_rows = 0;
  int max_seq_len = 0;   // longest context (after this step) in the batch
  int max_new_tokens = 0;  // longest portion
  bool decode_only = false;  // every request brings exactly one token
};

// Checks the entries against the manager (known ids, pages reserved for every token), writes the
// flat arrays into `staging` (layout.total int32s) and returns the counts. With `pad`, unused
// request rows and token rows up to the capacities are filled with a harmless request that owns
// only the null page `num_pages(g)` and the null slot `num_slots`, so that kernels launched for
// the full capacity (CUDA-graph replays) touch nothing that belongs to a live request.
StepCounts fill_step(const CacheManager& cm, const std::vector<StepEntry>& entries, const StepLayout& layout,
                     std::int32_t* staging, bool pad, int vocab_size, int max_positions);

}  // namespace llmhost

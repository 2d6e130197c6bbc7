#include "cache_manager.hpp"

#include <algorithm>
#include <cstring>
#include <stdexcept>

namespace llmhost {

CacheManager::CacheManager(int page_size, std::vector<GroupSpec> groups, int num_slots)
    : page_size_(page_size), num_slots_(num_slots) {
  if (page_size <= 0) throw std::invalid_argument("CacheManager: page_size must be >= 1");
  if (num_slots <= 0) throw std::invalid_argument("CacheManager: num_slots must be >= 1");
  if (groups.empty()) throw std::invalid_argument("CacheManager: at least one cache group is needed");
  for (const auto& g : groups) {
    if (g.num_pages <= 0) throw std::invalid_argument("CacheManager: num_pages must be >= 1");
    if (g.window < 0) throw std::invalid_argument("CacheManager: window must be >= 0");
    Group grp;
    grp.spec = g;
    for (int p = 0; p < g.num_pages; ++p) grp.free_list.push_back(p);
    groups_.push_back(std::move(grp));
  }
  for (int s = 0; s < num_slots; ++s) free_slots_.push_back(s);
}

const CacheManager::Group& CacheManager::group(int g) const {
  if (g < 0 || g >= static_cast<int>(groups_.size())) throw std::out_of_range("CacheManager: no such cache group");
  return groups_[g];
}

const CacheManager::Request& CacheManager::req(std::int64_t id) const {
  auto it = requests_.find(id);
  if (it == requests_.end()) throw std::out_of_range("CacheManager: unknown request " + std::to_string(id));
  return it->second;
}

CacheManager::Request& CacheManager::req(std::int64_t id) {
  return const_cast<Request&>(static_cast<const CacheManager*>(this)->req(id));
}

int CacheManager::add_request(std::int64_t id) {
  if (requests_.count(id)) throw std::invalid_argument("CacheManager: request " + std::to_string(id) + " already exists");
  if (free_slots_.empty()) return -1;
  Request r;
  r.slot = free_slots_.front();
  free_slots_.pop_front();
  r.tables.resize(groups_.size());
  requests_.emplace(id, std::move(r));
  return requests_.at(id).slot;
}

bool CacheManager::reserve(std::int64_t id, int n_new) {
  if (n_new < 0) throw std::invalid_argument("CacheManager::reserve: negative token count");
  Request& r = req(id);
  const int target_pages = pages_for(r.length + n_new);
  for (std::size_t g = 0; g < groups_.size(); ++g) {
    const int need = target_pages - static_cast<int>(r.tables[g].size());
    if (need > static_cast<int>(groups_[g].free_list.size())) return false;
  }
  for (std::size_t g = 0; g < groups_.size(); ++g) {
    while (static_cast<int>(r.tables[g].size()) < target_pages) {
      r.tables[g].push_back(groups_[g].free_list.front());
      groups_[g].free_list.pop_front();
    }
  }
  r.reserved = std::max(r.reserved, r.length + n_new);
  return true;
}

void CacheManager::advance(std::int64_t id, int n) {
  if (n < 0) throw std::invalid_argument("CacheManager::advance: negative token count");
  Request& r = req(id);
  if (r.length + n > r.reserved)
    throw std::logic_error("CacheManager::advance: request " + std::to_string(id) + " advances past its reserved pages");
  r.length += n;
  for (std::size_t g = 0; g < groups_.size(); ++g) {
    const int w = groups_[g].spec.window;
    if (w <= 0) continue;
    const int first_needed = r.length - w + 1;  // oldest key a later query can still read
    if (first_needed <= 0) continue;
    const int dead_pages = std::min<int>(first_needed / page_size_, static_cast<int>(r.tables[g].size()));
    for (int i = 0; i < dead_pages; ++i) {
      int& page = r.tables[g][i];
      if (page >= 0) {
        groups_[g].free_list.push_back(page);
        page = -1;
      }
    }
  }
}

void CacheManager::release(std::int64_t id) {
  auto it = requests_.find(id);
  if (it == requests_.end()) throw std::out_of_range("CacheManager::release: unknown request " + std::to_string(id));
  Request& r = it->second;
  for (std::size_t g = 0; g < groups_.size(); ++g)
    for (int page : r.tables[g])
      if (page >= 0) groups_[g].free_list.push_back(page);
  free_slots_.push_back(r.slot);
  requests_.erase(it);
}

const std::vector<int>& CacheManager::block_table(std::int64_t id, int g) const {
  group(g);
  return req(id).tables[g];
}

std::vector<std::int64_t> CacheManager::request_ids() const {
  std::vector<std::int64_t> out;
  for (const auto& kv : requests_) out.push_back(kv.first);
  return out;
}

void CacheManager::check() const {
  for (std::size_t g = 0; g < groups_.size(); ++g) {
    const int n = groups_[g].spec.num_pages;
    std::vector<int> owner(n, 0);  // 0 unseen, 1 free, 2 held
    auto mark = [&](int page, int kind, const std::string& who) {
      if (page < 0 || page >= n)
        throw std::logic_error("cache group " + std::to_string(g) + ": page id " + std::to_string(page) + " out of range (" + who + ")");
      if (owner[page] != 0)
        throw std::logic_error("cache group " + std::to_string(g) + ": page " + std::to_string(page) +
                               (owner[page] == 1 ? " is on the free list and also " : " is held and also ") + who);
      owner[page] = kind;
    };
    for (int page : groups_[g].free_list) mark(page, 1, "on the free list");
    for (const auto& kv : requests_) {
      const Request& r = kv.second;
      const auto& t = r.tables[g];
      if (static_cast<int>(t.size()) * page_size_ < r.reserved)
        throw std::logic_error("request " + std::to_string(kv.first) + ": block table shorter than its reserved length");
      if (r.length > r.reserved) throw std::logic_error("request " + std::to_string(kv.first) + ": length beyond reserved");
      const int w = groups_[g].spec.window;
      const int first_needed = w > 0 ? std::max(0, r.length - w + 1) : 0;
      for (std::size_t i = 0; i < t.size(); ++i) {
        if (t[i] >= 0) mark(t[i], 2, "held by request " + std::to_string(kv.first));
        else if (w <= 0 || static_cast<int>(i + 1) * page_size_ > first_needed)
          throw std::logic_error("request " + std::to_string(kv.first) + ": a page that is still needed was given back");
      }
    }
    for (int p = 0; p < n; ++p)
      if (owner[p] == 0) throw std::logic_error("cache group " + std::to_string(g) + ": page " + std::to_string(p) + " is lost");
  }
  std::vector<int> slot_owner(num_slots_, 0);
  auto mark_slot = [&](int s, const std::string& who) {
    if (s < 0 || s >= num_slots_) throw std::logic_error("slot id out of range (" + who + ")");
    if (slot_owner[s]++) throw std::logic_error("slot " + std::to_string(s) + " is held twice (" + who + ")");
  };
  for (int s : free_slots_) mark_slot(s, "free list");
  for (const auto& kv : requests_) mark_slot(kv.second.slot, "request " + std::to_string(kv.first));
  for (int s = 0; s < num_slots_; ++s)
    if (!slot_owner[s]) throw std::logic_error("slot " + std::to_string(s) + " is lost");
}

// ------------------------------------------------------------------------------------------------
static int align4(int x) { return (x + 3) & ~3; }

StepLayout StepLayout::make(int cap_tokens, int cap_seqs, int cap_rows, int max_blocks, int num_groups) {
  if (cap_tokens <= 0 || cap_seqs <= 0 || cap_rows < 0 || max_blocks <= 0 || num_groups <= 0)
    throw std::invalid_argument("StepLayout: capacities must be positive");
  StepLayout l;
  l.cap_tokens = cap_tokens; l.cap_seqs = cap_seqs; l.cap_rows = cap_rows; l.max_blocks = max_blocks;
  l.num_groups = num_groups;
  int off = 0;
  auto take = [&](int n) { int o = off; off = align4(off + n); return o; };
  l.token_ids = take(cap_tokens);
  l.positions = take(cap_tokens);
  l.token_seq = take(cap_tokens);
  l.logit_rows = take(cap_rows);
  l.row_temperature = take(cap_rows);
  l.row_seed = take(cap_rows);
  l.row_draw = take(cap_rows);
  l.seq_start = take(cap_seqs);
  l.seq_ntok = take(cap_seqs);
  l.seq_qoff = take(cap_seqs + 1);
  l.seq_slot = take(cap_seqs);
  l.seq_len = take(cap_seqs);
  l.block_tables = take(num_groups * cap_seqs * max_blocks);
  l.total = off;
  return l;
}

StepCounts fill_step(const CacheManager& cm, const std::vector<StepEntry>& entries, const StepLayout& L,
                     std::int32_t* s, bool pad, int vocab_size, int max_positions) {
  if (L.num_groups != cm.num_groups()) throw std::invalid_argument("fill_step: layout and cache manager disagree on groups");
  StepCounts c;
  c.n_seqs = static_cast<int>(entries.size());
  if (c.n_seqs > L.cap_seqs) throw std::invalid_argument("fill_step: more requests than the layout's capacity");
  c.decode_only = c.n_seqs > 0;
  int tok = 0, row = 0;
  for (int i = 0; i < c.n_seqs; ++i) {
    const StepEntry& e = entries[i];
    const int n = static_cast<int>(e.tokens.size());
    if (n == 0) throw std::invalid_argument("step: request " + std::to_string(e.id) + " brings no tokens");
    for (int j = 0; j < i; ++j)
      if (entries[j].id == e.id) throw std::invalid_argument("step: request " + std::to_string(e.id) + " appears twice");
    if (!cm.has_request(e.id)) throw std::invalid_argument("step: unknown request " + std::to_string(e.id));
    const int start = cm.length(e.id);
    if (start + n > cm.reserved(e.id))
      throw std::logic_error("step: request " + std::to_string(e.id) + " has no pages reserved for its tokens");
    if (start + n > max_positions)
      throw std::invalid_argument("step: request " + std::to_string(e.id) + " would exceed the position limit " +
                                  std::to_string(max_positions));
    if (tok + n > L.cap_tokens) throw std::invalid_argument("fill_step: more tokens than the layout's capacity");
    if (n != 1) c.decode_only = false;
    s[L.seq_start + i] = start;
    s[L.seq_ntok + i] = n;
    s[L.seq_qoff + i] = tok;
    s[L.seq_slot + i] = cm.slot(e.id);
    s[L.seq_len + i] = start + n;
    c.max_seq_len = std::max(c.max_seq_len, start + n);
    c.max_new_tokens = std::max(c.max_new_tokens, n);
    for (int j = 0; j < n; ++j) {
      const std::int32_t t = e.tokens[j];
      if (t < 0 || t >= vocab_size)
        throw std::invalid_argument("step: token id " + std::to_string(t) + " out of range [0, " + std::to_string(vocab_size) + ")");
      s[L.token_ids + tok + j] = t;
      s[L.positions + tok + j] = start + j;
      s[L.token_seq + tok + j] = i;
    }
    for (std::int32_t wv : e.want) {
      if (wv < 0 || wv >= n) throw std::invalid_argument("step: wanted place " + std::to_string(wv) + " is not among the request's tokens");
      if (row >= L.cap_rows) throw std::invalid_argument("fill_step: more wanted rows than the layout's capacity");
      s[L.logit_rows + row] = tok + wv;
      std::memcpy(&s[L.row_temperature + row], &e.temperature, sizeof(float));
      s[L.row_seed + row] = e.seed;
      s[L.row_draw + row] = e.draw;
      ++row;
    }
    for (int g = 0; g < L.num_groups; ++g) {
      const auto& t = cm.block_table(e.id, g);
      if (static_cast<int>(t.size()) > L.max_blocks) throw std::invalid_argument("fill_step: block table wider than the layout");
      std::int32_t* dst = s + L.block_tables + (static_cast<std::size_t>(g) * L.cap_seqs + i) * L.max_blocks;
      std::size_t k = 0;
      for (; k < t.size(); ++k) dst[k] = t[k];
      for (; k < static_cast<std::size_t>(L.max_blocks); ++k) dst[k] = -1;
    }
    tok += n;
  }
  s[L.seq_qoff + c.n_seqs] = tok;
  c.n_tokens = tok;
  c.n_rows = row;
  if (pad) {
    // the remaining request rows each bring one token at position 0 of the null page
    int i = c.n_seqs;
    for (; i < L.cap_seqs && tok < L.cap_tokens; ++i, ++tok) {
      s[L.seq_start + i] = 0;
      s[L.seq_ntok + i] = 1;
      s[L.seq_qoff + i] = tok;
      s[L.seq_slot + i] = cm.num_slots();
      s[L.seq_len + i] = 1;
      s[L.token_ids + tok] = 0;
      s[L.positions + tok] = 0;
      s[L.token_seq + tok] = i;
      for (int g = 0; g < L.num_groups; ++g) {
        std::int32_t* dst = s + L.block_tables + (static_cast<std::size_t>(g) * L.cap_seqs + i) * L.max_blocks;
        for (int k = 0; k < L.max_blocks; ++k) dst[k] = cm.num_pages(g);
      }
    }
    s[L.seq_qoff + i] = tok;
    for (int r = row; r < L.cap_rows; ++r) {
      s[L.logit_rows + r] = 0;
      s[L.row_temperature + r] = 0;
      s[L.row_seed + r] = 0;
      s[L.row_draw + r] = 0;
    }
  }
  return c;
}

}  // namespace llmhost

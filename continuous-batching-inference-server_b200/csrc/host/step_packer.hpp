// Packs the description of a step into one int32 buffer (pinned host memory, copied to the device in
// one piece): tokens, positions, the segment of each row, segment tables, the rows whose logits are
// wanted, and per cache group the token slots and the block tables of the step's requests.
//
// The reference builds per-ROW arrays on the host and copies a whole 2048-entry page table per row
// (src/transformer.cpp:51-63).  Here a step is a list of segments; single-token segments (decoding)
// are ordered first; block tables go per REQUEST.
#pragma once
#include <algorithm>
#include <cstdint>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

#include "cache_manager.hpp"
#include "scheduler.hpp"

namespace cbis {

struct PackEntry {
  int slot = 0;
  int start = 0;
  std::vector<int> tokens;
  std::vector<int> want;  // places among `tokens` whose logits are wanted
};

struct PackInfo {
  int n_rows = 0, n_segments = 0, n_logit_rows = 0, n_decode = 0, max_seg_rows = 0, max_ctx = 0;
  int n_tokens = 0;        // tokens of the entries (n_rows counts the padding rows of a fixed-size step too)
  int n_wanting = 0;       // entries that want logits at one place or more
  int n_wanted = 0;        // places at which logits are wanted (n_logit_rows counts the padding of a fixed-size step too)
  std::vector<int> seg_rows, seg_ctx;  // per segment, in the step's order (padding segments included)
};

class StepPacker {
 public:
  StepPacker(const CacheManager* cache, int max_tokens, int max_seqs, int vocab, int max_positions,
             std::vector<int> max_blocks, int n_groups)
      : cache_(cache), T_(max_tokens), S_(max_seqs), vocab_(vocab), pmax_(max_positions),
        max_blocks_(std::move(max_blocks)), n_groups_(n_groups) {
    int off = 0;
    auto field = [&](const std::string& name, int n) {
      layout_[name] = {off, n};
      off += (n + 3) / 4 * 4;  // fields start on 16-byte boundaries
    };
    for (const char* name : {"tokens", "positions", "row_seq", "logit_rows"}) field(name, T_);
    for (const char* name : {"seg_slot", "seg_start", "seg_ctx"}) field(name, S_);
    field("cu_rows", S_ + 1);
    for (int g = 0; g < n_groups_; ++g) {
      field("slot_mapping" + std::to_string(g), T_);
      field("block_table" + std::to_string(g), S_ * max_blocks_.at(g));
    }
    words_ = off;
  }

  int words() const { return words_; }
  const std::map<std::string, std::pair<int, int>>& layout() const { return layout_; }

  PackInfo pack_plan(uintptr_t buffer, const std::vector<PlannedEntry>& plan, int pad_rows, bool all_logits,
                     int pad_segments = 0) const {
    std::vector<PackEntry> es(plan.size());
    for (size_t i = 0; i < plan.size(); ++i) {
      es[i].slot = plan[i].slot;
      es[i].start = plan[i].start;
      es[i].tokens = plan[i].tokens;
      if (plan[i].sample) es[i].want.push_back((int)plan[i].tokens.size() - 1);
    }
    return pack(buffer, es, pad_rows, all_logits, false, pad_segments);
  }

  // `reserved_ahead`: the cache may already hold room beyond the step's tokens (a run of decode steps
  // whose pages were taken beforehand).
  // `pad_rows` alone: a step of single tokens laid out for exactly that many rows and segments (rows beyond the
  // entries belong to no segment).  With `pad_segments`: any step laid out for pad_rows rows, pad_segments segments
  // (those beyond the entries hold no rows) and pad_segments wanted rows (those beyond the entries' repeat row 0);
  // it counts as a step without one-token segments, so that every segment goes the way of the longer ones.
  PackInfo pack(uintptr_t buffer, const std::vector<PackEntry>& entries, int pad_rows, bool all_logits,
                bool reserved_ahead, int pad_segments = 0) const {
    validate(entries, reserved_ahead);
    int32_t* buf = reinterpret_cast<int32_t*>(buffer);
    auto at = [&](const std::string& name) { return buf + layout_.at(name).first; };
    const int n = (int)entries.size();
    std::vector<int> order(n);
    for (int i = 0; i < n; ++i) order[i] = i;
    std::stable_sort(order.begin(), order.end(),
                     [&](int a, int b) { return (entries[a].tokens.size() != 1) < (entries[b].tokens.size() != 1); });
    int32_t *tokens = at("tokens"), *positions = at("positions"), *row_seq = at("row_seq");
    int32_t *seg_slot = at("seg_slot"), *seg_start = at("seg_start"), *seg_ctx = at("seg_ctx"), *cu = at("cu_rows");
    std::vector<int> row0(n);
    PackInfo info;
    int r = 0;
    cu[0] = 0;
    for (int s = 0; s < n; ++s) {
      const PackEntry& e = entries[order[s]];
      const int k = (int)e.tokens.size();
      row0[order[s]] = r;
      for (int i = 0; i < k; ++i) {
        tokens[r + i] = e.tokens[i];
        positions[r + i] = e.start + i;
        row_seq[r + i] = s;
      }
      seg_slot[s] = e.slot;
      seg_start[s] = e.start;
      seg_ctx[s] = e.start + k;
      info.seg_rows.push_back(k);
      info.seg_ctx.push_back(e.start + k);
      info.n_decode += k == 1;
      r += k;
      cu[s + 1] = r;
    }
    int T = r, S = n;
    const int real_rows = T, real_segs = S;
    if (pad_rows > 0 && pad_segments > 0) {
      if (pad_rows < T || pad_rows > T_ || pad_segments < n || pad_segments > S_ || all_logits)
        throw std::invalid_argument("a step laid out for fixed sizes must fit them");
      for (int i = T; i < pad_rows; ++i) {
        tokens[i] = 0;
        positions[i] = 0;
        row_seq[i] = -1;
      }
      for (int s = S; s < pad_segments; ++s) {
        seg_slot[s] = seg_start[s] = seg_ctx[s] = 0;
        cu[s + 1] = real_rows;
        info.seg_rows.push_back(0);
        info.seg_ctx.push_back(0);
      }
      T = pad_rows;
      S = pad_segments;
      info.n_decode = 0;
    } else if (pad_rows > 0) {
      if (info.n_decode != n || pad_rows < n || pad_rows > T_ || pad_rows > S_)
        throw std::invalid_argument("a padded step holds single tokens only and fits the engine's limits");
      for (int i = T; i < pad_rows; ++i) {
        tokens[i] = 0;
        positions[i] = 0;
        row_seq[i] = -1;
      }
      for (int s = S; s < pad_rows; ++s) {
        seg_slot[s] = seg_start[s] = seg_ctx[s] = 0;
        info.seg_rows.push_back(1);
        info.seg_ctx.push_back(0);
      }
      for (int s = 0; s <= pad_rows; ++s) cu[s] = std::min(s, real_rows);
      T = S = pad_rows;
      info.n_decode = pad_rows;
    }
    int32_t* logit_rows = at("logit_rows");
    int R = 0;
    if (all_logits) {
      for (int i = 0; i < T; ++i) logit_rows[R++] = i;
    } else {
      for (int i = 0; i < n; ++i)
        for (int w : entries[i].want) logit_rows[R++] = row0[i] + w;
    }
    info.n_wanted = all_logits ? real_rows : R;
    if (pad_segments > 0) {
      if (R > pad_segments) throw std::invalid_argument("a step laid out for fixed sizes wants at most one row per segment");
      while (R < pad_segments) logit_rows[R++] = 0;
    }
    for (int g = 0; g < n_groups_; ++g) {
      const int ps = cache_->page_size(g), mb = max_blocks_[g];
      int32_t* sm = at("slot_mapping" + std::to_string(g));
      int32_t* bt = at("block_table" + std::to_string(g));
      for (int s = 0; s < S; ++s) {
        int32_t* row = bt + (size_t)s * mb;
        if (s >= real_segs) {
          std::fill(row, row + mb, -1);
          continue;
        }
        const PackEntry& e = entries[order[s]];
        const std::vector<int>& table = cache_->block_table(e.slot, g);
        const int have = std::min<int>((int)table.size(), mb);
        std::copy(table.begin(), table.begin() + have, row);
        std::fill(row + have, row + mb, -1);
        for (int i = cu[s]; i < (s + 1 <= real_segs ? (int)cu[s + 1] : cu[s]); ++i) {
          const int pos = positions[i];
          const int page = pos / ps < have ? table[pos / ps] : -1;
          sm[i] = page >= 0 ? page * ps + pos % ps : -1;
        }
      }
      for (int i = real_rows; i < T; ++i) sm[i] = -1;
    }
    info.n_rows = T;
    info.n_tokens = real_rows;
    for (const auto& e : entries) info.n_wanting += !e.want.empty();
    info.n_segments = S;
    info.n_logit_rows = R;
    info.max_seg_rows = *std::max_element(info.seg_rows.begin(), info.seg_rows.end());
    info.max_ctx = *std::max_element(info.seg_ctx.begin(), info.seg_ctx.end());
    return info;
  }

 private:
  void validate(const std::vector<PackEntry>& entries, bool reserved_ahead) const {
    if (entries.empty()) throw std::invalid_argument("a step needs at least one entry");
    if ((int)entries.size() > S_)
      throw std::invalid_argument(std::to_string(entries.size()) + " requests in one step; the engine was made for " +
                                  std::to_string(S_));
    long total = 0;
    for (const auto& e : entries) total += (long)e.tokens.size();
    if (total > T_)
      throw std::invalid_argument(std::to_string(total) + " tokens in one step; the engine was made for " +
                                  std::to_string(T_));
    std::vector<char> seen(cache_->max_requests(), 0);
    for (const auto& e : entries) {
      const int k = (int)e.tokens.size();
      const std::string who = "slot " + std::to_string(e.slot);
      if (k == 0) throw std::invalid_argument(who + ": an entry without tokens");
      if (!cache_->live(e.slot)) throw std::invalid_argument(who + " holds no request");
      if (seen[e.slot]) throw std::invalid_argument(who + " appears twice in one step");
      seen[e.slot] = 1;
      if (e.start < 0 || e.start + k > pmax_)
        throw std::invalid_argument(who + ": positions " + std::to_string(e.start) + ".." + std::to_string(e.start + k - 1) +
                                    " exceed the model's " + std::to_string(pmax_) + " positions");
      const int len = cache_->length(e.slot);
      if (!(reserved_ahead ? len >= e.start + k : len == e.start + k))
        throw std::invalid_argument(who + ": the cache holds room for " + std::to_string(len) +
                                    " tokens, the step brings tokens " + std::to_string(e.start) + ".." +
                                    std::to_string(e.start + k - 1));
      for (int t : e.tokens)
        if (t < 0 || t >= vocab_)
          throw std::invalid_argument(who + ": token id " + std::to_string(t) + " outside the vocabulary of " +
                                      std::to_string(vocab_));
      for (int w : e.want)
        if (w < 0 || w >= k)
          throw std::invalid_argument(who + ": wanted place " + std::to_string(w) + " outside its " + std::to_string(k) +
                                      " tokens");
    }
  }

  const CacheManager* cache_;
  int T_, S_, vocab_, pmax_;
  std::vector<int> max_blocks_;
  int n_groups_;
  std::map<std::string, std::pair<int, int>> layout_;
  int words_ = 0;
};

}  // namespace cbis

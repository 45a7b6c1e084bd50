// Continuous-batching scheduler: admits requests, cuts prompts into portions under a token
// budget, decodes, finishes and frees; preempts when pages run out.
//
// The reference's loop (src/server_demo.cpp:129-185, src/bench_batching.cpp:98-179) admits
// FIFO into free slots, feeds a new request's whole prompt in one step beside one decode
// token per running request, samples on each request's last row, finishes after decode_len
// outputs and frees the pages.  It has no token budget, and running out of pages ends the
// process (src/bench_batching.cpp:133,143).  Here:
//   * a step holds at most max_batched_tokens tokens and max_num_seqs requests;
//   * running requests go first, oldest first; a request needs `remaining` tokens fed
//     (1 while decoding), cut to min(remaining, prefill_chunk, budget left);
//   * when a running request cannot get pages, the most recently admitted running request is
//     preempted: its pages and slot are freed, it keeps its tokens (prompt and outputs so far)
//     and goes to the FRONT of the waiting queue, to be recomputed later; sampling is keyed
//     by (request, output index), so it continues as it would have;
//   * waiting requests are admitted FIFO while a slot, budget and pages for their first
//     portion are there; a request that could never fit is refused when it is added;
//   * the step after a launched one can be planned before that one's tokens are known (schedule_ahead), when it is
//     certain but for the tokens: decoding goes on for everyone whatever is sampled, short of an end-of-sequence
//     token, and then the request's row of the step planned ahead is computed for nothing;
//   * a step that preempted admits nobody, and a request that was preempted before comes back
//     only when everything it holds so far, plus a page, fits beside the running requests:
//     otherwise the pages it just gave up would let it in again at once, to be recomputed and
//     thrown out again every few steps.
#pragma once
#include <algorithm>
#include <cstdint>
#include <deque>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "cache_manager.hpp"

namespace cbis {

struct SchedulerLimits {
  int max_num_seqs = 16;          // reference: kMaxSlots (src/server_demo.cpp:27)
  int max_batched_tokens = 512;   // reference: kMaxTotalRows (src/server_demo.cpp:29)
  int prefill_chunk = 512;        // reference: 512-row portions in src/bench_tiering.cpp:78
  int max_positions = 0;          // the model's position limit
};

struct PlannedEntry {
  int64_t request_id;
  int slot;
  int start;                 // position of the first token of this portion
  std::vector<int> tokens;   // the tokens to run
  bool sample;               // the portion ends the known tokens: its last row yields the next token
  int output_index;          // index of the token that will be sampled (for the sampling key)
  bool ahead = false;        // planned by schedule_ahead: the one token is a placeholder, the step before samples it
  int source = -1;           // ahead: which of the step before's sampled tokens (in its sampling entries' order) it is
};

struct Finished {
  int64_t request_id;
  std::string reason;        // "length" (max_new_tokens or position limit) or "stop" (eos)
  std::vector<int> output;
};

class Scheduler {
 public:
  Scheduler(CacheManager* cache, SchedulerLimits lim) : cache_(cache), lim_(lim) {
    if (lim.max_num_seqs <= 0 || lim.max_batched_tokens <= 0 || lim.prefill_chunk <= 0 || lim.max_positions <= 0)
      throw std::invalid_argument("Scheduler: limits must be positive");
  }

  void add(int64_t id, std::vector<int> prompt, int max_new_tokens, int eos_token, bool ignore_eos) {
    if (reqs_.count(id)) throw std::invalid_argument("request " + std::to_string(id) + " exists already");
    if (prompt.empty()) throw std::invalid_argument("request " + std::to_string(id) + ": empty prompt");
    if (max_new_tokens <= 0) throw std::invalid_argument("request " + std::to_string(id) + ": max_new_tokens must be positive");
    if ((int)prompt.size() > lim_.max_positions)
      throw std::invalid_argument("request " + std::to_string(id) + ": prompt of " + std::to_string(prompt.size()) +
                                  " tokens exceeds the model's " + std::to_string(lim_.max_positions) + " positions");
    // Tokens the cache must hold at most: all fed tokens; the last output is never fed back.
    const long most = std::min<long>((long)prompt.size() + max_new_tokens - 1, lim_.max_positions);
    if (!cache_->fits_at_all((int)most, std::min(lim_.prefill_chunk, lim_.max_batched_tokens)))
      throw std::invalid_argument("request " + std::to_string(id) + ": " + std::to_string(most) +
                                  " tokens can never fit into the cache pool");
    Req r;
    r.id = id;
    r.prompt_len = (int)prompt.size();
    r.tokens = std::move(prompt);
    r.max_new = max_new_tokens;
    r.eos = eos_token;
    r.ignore_eos = ignore_eos;
    reqs_.emplace(id, std::move(r));
    waiting_.push_back(id);
  }

  bool abort(int64_t id) {
    auto it = reqs_.find(id);
    if (it == reqs_.end()) return false;
    if (it->second.slot >= 0) cache_->release(it->second.slot);
    running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
    waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), id), waiting_.end());
    reqs_.erase(it);
    return true;
  }

  int num_waiting() const { return (int)waiting_.size(); }
  int num_running() const { return (int)running_.size(); }
  bool idle() const { return waiting_.empty() && running_.empty(); }
  long preemptions() const { return preemptions_; }
  std::vector<int64_t> running_ids() const { return running_; }
  std::vector<int64_t> waiting_ids() const { return {waiting_.begin(), waiting_.end()}; }

  // Decides the next step.  Pages for every planned portion are taken here.  An empty plan
  // with requests left means nothing can run now (cannot happen while a request is running).
  std::vector<PlannedEntry> schedule() {
    if (pending_ > 0) throw std::logic_error("schedule: the tokens of the step before have not come back (update)");
    std::vector<PlannedEntry> plan;
    int budget = lim_.max_batched_tokens;
    // Pages behind a window are given back only now: the step that was planned last still read
    // them, and it has been launched (work on the device runs in launch order).
    for (int64_t id : running_) cache_->release_out_of_window(reqs_.at(id).slot);
    // (1) running requests, oldest first
    const long preemptions_before = preemptions_;
    for (size_t i = 0; i < running_.size() && budget > 0;) {
      Req& r = reqs_.at(running_[i]);
      const int remaining = (int)r.tokens.size() - r.computed;
      int n = std::min({remaining, remaining == 1 ? 1 : lim_.prefill_chunk, budget});
      bool skipped = false;
      while (true) {
        const int fit = cache_->max_appendable(r.slot, n);
        if (fit >= n) break;
        if (running_.size() - 1 > i) {  // someone newer holds pages: take them
          preempt(running_.back());
          continue;
        }
        // r is the newest running request
        if (fit >= 1 && remaining > 1) { n = fit; break; }        // a smaller portion of the prompt
        if (i == 0) throw std::logic_error("scheduler: a request alone does not fit; add() should have refused it");
        skipped = true;                                            // wait for older requests to finish
        break;
      }
      if (skipped) { ++i; continue; }
      emit(r, n, &plan);
      budget -= n;
      ++i;
    }
    // (2) admissions, FIFO
    while (preemptions_ == preemptions_before && !waiting_.empty() && budget > 0 &&
           (int)running_.size() < lim_.max_num_seqs && cache_->free_slots() > 0) {
      Req& r = reqs_.at(waiting_.front());
      const int remaining = (int)r.tokens.size();
      int n = std::min({remaining, lim_.prefill_chunk, budget});
      // preempted before: room for all it knows and a page more (one token more per group rounds up to that)
      if (r.times_preempted > 0 && !running_.empty() && !cache_->fits_fresh(remaining + cache_->largest_page()))
        break;
      if (!cache_->fits_fresh(n)) {
        if (!running_.empty()) break;  // wait until running requests give pages back
        // nothing is running, so every page is free: take what fits (add() made sure it can finish)
        int fit = n;
        while (fit > 0 && !cache_->fits_fresh(fit)) --fit;
        if (fit == 0) throw std::logic_error("scheduler: empty cache cannot hold one token");
        n = fit;
      }
      const int slot = cache_->admit(r.id);
      if (slot < 0) break;
      waiting_.pop_front();
      r.slot = slot;
      r.computed = 0;
      r.admitted_now = true;
      running_.push_back(r.id);
      emit(r, n, &plan);
      budget -= n;
    }
    remember_sampling(plan);
    return plan;
  }

  // Plans the step AFTER one whose sampled tokens are still on their way (schedule() or schedule_ahead() has been
  // called and the update has not), if that step is certain but for its tokens: every running request waits for
  // exactly one sampled token and goes on decoding whatever it is (it reaches neither its output limit nor the
  // position limit with it; only an end-of-sequence token can stop it, and then its row of this step is computed
  // for nothing and update_plan passes over it), nobody waits for admission, and pages for one more token each are
  // free.  Otherwise an empty plan, and nothing has changed: the caller updates first and calls schedule().
  // The entries hold a placeholder token (0): the device has the real one, `source` says which of the step before's
  // sampled tokens it is (a request of that step may have ended meanwhile, so the rows need not line up).
  std::vector<PlannedEntry> schedule_ahead() {
    std::vector<PlannedEntry> plan;
    if (pending_ != 1 || running_.empty() || !waiting_.empty() || (int)running_.size() > lim_.max_batched_tokens)
      return plan;
    for (int64_t id : running_) {
      const Req& r = reqs_.at(id);
      const int size = (int)r.tokens.size();
      if (r.computed != size) return plan;                                   // tokens still to be fed, or already a step ahead
      if (size + 1 - r.prompt_len >= r.max_new || size + 1 > lim_.max_positions) return plan;   // ends with the token on its way
    }
    for (int64_t id : running_) cache_->release_out_of_window(reqs_.at(id).slot);   // the step before has been launched
    for (int g = 0; g < cache_->num_groups(); ++g) {
      long need = 0;
      for (int64_t id : running_) need += cache_->pages_needed(reqs_.at(id).slot, g, 1);
      if (need > cache_->free_pages(g)) return plan;
    }
    for (int64_t id : running_) {
      Req& r = reqs_.at(id);
      if (!cache_->append(r.slot, 1)) throw std::logic_error("scheduler: pages vanished between check and take");
      PlannedEntry e;
      e.request_id = r.id;
      e.slot = r.slot;
      e.start = r.computed;
      e.tokens.assign(1, 0);
      e.sample = true;
      e.output_index = (int)r.tokens.size() + 1 - r.prompt_len;
      e.ahead = true;
      const auto at = std::find(last_sampling_.begin(), last_sampling_.end(), r.id);
      if (at == last_sampling_.end()) throw std::logic_error("schedule_ahead: a request awaits a token no step samples");
      e.source = (int)(at - last_sampling_.begin());
      r.computed += 1;
      plan.push_back(std::move(e));
    }
    remember_sampling(plan);
    return plan;
  }

  // The `source` of every entry of the plan that schedule_ahead() made last; empty if entry i takes token i.
  std::vector<int> ahead_sources() const { return ahead_sources_; }

  // Slots admitted by the last schedule() call; their fixed-size state must be cleared before the step.
  std::vector<int> take_new_slots() {
    std::vector<int> out;
    for (int64_t id : running_) {
      Req& r = reqs_.at(id);
      if (r.admitted_now) { out.push_back(r.slot); r.admitted_now = false; }
    }
    return out;
  }

  // The same with the plan itself: `tokens` holds one token for every entry of the plan that samples, in the plan's order.
  std::vector<Finished> update_plan(const std::vector<PlannedEntry>& plan, const std::vector<int>& tokens) {
    std::vector<std::pair<int64_t, int>> sampled;
    sampled.reserve(tokens.size());
    size_t k = 0;
    for (const auto& e : plan) {
      if (!e.sample) continue;
      if (k >= tokens.size()) throw std::invalid_argument("update_plan: fewer tokens than sampling entries");
      // a request that ended (or was aborted) while its step planned ahead was on its way: that row was for nothing
      if (e.ahead && !reqs_.count(e.request_id)) { ++k; continue; }
      sampled.emplace_back(e.request_id, tokens[k++]);
    }
    if (k != tokens.size()) throw std::invalid_argument("update_plan: more tokens than sampling entries");
    return update(sampled);
  }

  // Takes the sampled tokens of the last step, in the order of the plan's sampling entries.
  std::vector<Finished> update(const std::vector<std::pair<int64_t, int>>& sampled) {
    std::vector<Finished> done;
    if (pending_ > 0) --pending_;
    for (const auto& [id, tok] : sampled) {
      auto it = reqs_.find(id);
      if (it == reqs_.end()) throw std::invalid_argument("update: unknown request " + std::to_string(id));
      Req& r = it->second;
      // all known tokens have been run, and with a step planned ahead the one that arrives now has been too
      if (r.computed != (int)r.tokens.size() && r.computed != (int)r.tokens.size() + 1)
        throw std::logic_error("update: request has tokens not yet run");
      r.tokens.push_back(tok);
      const int generated = (int)r.tokens.size() - r.prompt_len;
      std::string reason;
      if (!r.ignore_eos && r.eos >= 0 && tok == r.eos) reason = "stop";
      else if (generated >= r.max_new) reason = "length";            // src/server_demo.cpp:181
      else if ((int)r.tokens.size() > lim_.max_positions) reason = "length";  // no position left to feed it at
      if (!reason.empty()) {
        Finished f;
        f.request_id = id;
        f.reason = reason;
        f.output.assign(r.tokens.begin() + r.prompt_len, r.tokens.end());
        done.push_back(std::move(f));
        cache_->release(r.slot);
        running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
        reqs_.erase(it);
      }
    }
    return done;
  }

 private:
  struct Req {
    int64_t id = 0;
    std::vector<int> tokens;  // prompt followed by outputs so far
    int prompt_len = 0;
    int max_new = 0;
    int eos = -1;
    bool ignore_eos = false;
    int computed = 0;         // tokens whose keys/values are in the cache
    int slot = -1;
    bool admitted_now = false;
    int times_preempted = 0;
  };

  void emit(Req& r, int n, std::vector<PlannedEntry>* plan) {
    if (!cache_->append(r.slot, n)) throw std::logic_error("scheduler: pages vanished between check and take");
    PlannedEntry e;
    e.request_id = r.id;
    e.slot = r.slot;
    e.start = r.computed;
    e.tokens.assign(r.tokens.begin() + r.computed, r.tokens.begin() + r.computed + n);
    r.computed += n;
    e.sample = r.computed == (int)r.tokens.size();
    e.output_index = (int)r.tokens.size() - r.prompt_len;
    plan->push_back(std::move(e));
  }

  // Notes the requests that the plan samples for, in order; a plan that samples counts as open until its update.
  void remember_sampling(const std::vector<PlannedEntry>& plan) {
    std::vector<int64_t> ids;
    bool identity = true;
    ahead_sources_.clear();
    for (const PlannedEntry& e : plan) {
      if (!e.sample) continue;
      if (e.ahead) {
        identity = identity && e.source == (int)ids.size();
        ahead_sources_.push_back(e.source);
      }
      ids.push_back(e.request_id);
    }
    if (identity) ahead_sources_.clear();
    if (!ids.empty()) {
      ++pending_;
      last_sampling_ = std::move(ids);
    }
  }

  void preempt(int64_t id) {
    Req& r = reqs_.at(id);
    cache_->release(r.slot);
    r.slot = -1;
    r.computed = 0;
    r.admitted_now = false;
    ++r.times_preempted;
    running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
    waiting_.push_front(id);
    ++preemptions_;
  }

  CacheManager* cache_;
  SchedulerLimits lim_;
  std::unordered_map<int64_t, Req> reqs_;
  std::deque<int64_t> waiting_;
  std::vector<int64_t> running_;  // in admission order
  long preemptions_ = 0;
  int pending_ = 0;               // steps planned with sampling entries whose tokens have not come back yet
  std::vector<int64_t> last_sampling_;   // the requests the last such step samples for, in its entries' order
  std::vector<int> ahead_sources_;
};

}  // namespace cbis

// Continuous-batching scheduler: admits requests, cuts prompts into portions under a token
// budget, lets every running request decode each step, finishes and frees.
//
// Policy restated from the reference scheduler (crates/aien-scheduler/src/lib.rs):
//   * limits: max_batch_size sequences and max_batch_tokens tokens per step, max_prefill_tokens
//     of prompt per step, prefill_chunk_size per portion, watermark_blocks of headroom (:53-73);
//   * order of a step: watermark check (maybe preempt one) -> running requests in id order
//     (a decode token, or the next portion of the prompt) -> if nothing was preempted, admit
//     from the preempted queue first, then from the waiting queue, first come first served
//     (:733-1142);
//   * out of pages: the lowest-priority running request is preempted: its pages are given back
//     and it is queued to be recomputed from `prompt ++ generated`, so no token is emitted
//     twice (:741-779; crates/aien-scheduler/src/sequence.rs:318-323);
//   * a request ends on one of its stop ids (consumed, not emitted) or at max_tokens (:1349-1354).
// Own design: pages are allocated portion by portion; admission instead reserves, on paper,
// the pages of the whole input of every admitted request, so admitted work always completes.
#pragma once
#include <cstdint>
#include <deque>
#include <map>
#include <string>
#include <tuple>
#include <vector>

#include "cache_manager.h"

namespace pybind11 { class module_; }

namespace aien {

struct SchedulerConfig {
    int max_batch_size = 64;
    int max_batch_tokens = 4096;
    int max_prefill_tokens = 2048;
    int prefill_chunk_size = 512;
    bool chunk_prefill = true;
    int watermark_blocks = 4;
    int max_context = 0;        // 0: unlimited; else a request ends when it holds this many tokens
    // Own option, off at 0: a step that holds a portion of a longer input is cut so that its tokens fill whole
    // tiles of this many rows (the products work on 128 rows at a time: 536 rows cost what 640 do).  Only a
    // portion that is not its input's last is cut, and by a quarter of its length at most.
    int align_step_tokens = 0;
};

enum class SeqState : int { Waiting = 0, Running = 1, Preempted = 2, Finished = 3 };
enum class FinishReason : int { None = 0, StopToken = 1, LengthLimit = 2, Cancelled = 3, Aborted = 4 };

struct SeqRecord {
    int64_t id = 0;
    std::vector<int32_t> prompt;
    std::vector<int32_t> generated;
    int computed = 0;            // tokens of `prompt ++ generated` whose keys/values are cached
    int max_tokens = 0;
    std::vector<int32_t> stop_ids;
    int priority = 0;            // larger = more important
    uint64_t arrival = 0;
    int preemptions = 0;
    SeqState state = SeqState::Waiting;
    FinishReason reason = FinishReason::None;
    std::string message;
    int unresolved = 0;          // trailing tokens of `generated` whose values are not known yet (held as -1)
    bool draining = false;       // reached a length limit with a token unresolved: runs no more, ends at resolve()
    std::string drain_message;

    int input_len() const { return static_cast<int>(prompt.size() + generated.size()); }
    int32_t input_at(int i) const {
        return i < static_cast<int>(prompt.size()) ? prompt[i] : generated[i - prompt.size()];
    }
};

struct StepEntry {
    int64_t id = 0;
    std::vector<int32_t> tokens;
    int start = 0;               // position of tokens[0]
    bool wants_logits = false;   // the portion reaches the end of the input: sample after it
    uint64_t arrival = 0;        // which submission of this id the entry belongs to (ids may be used again)
};

struct StepPlan {
    int64_t step_id = 0;
    std::vector<StepEntry> entries;
    std::vector<int64_t> preempted;
    std::vector<PageCopy> copies;
    int num_tokens = 0;
    int prefill_tokens = 0;
};

struct FinishEvent {
    int64_t id = 0;
    FinishReason reason = FinishReason::None;
    std::vector<int32_t> generated;
    std::string message;
};

struct SchedulerMetrics {
    long long steps = 0, tokens_scheduled = 0, prefill_tokens = 0, decode_tokens = 0;
    long long preemptions = 0, finished = 0, admitted = 0;
};

class Scheduler {
  public:
    Scheduler(SchedulerConfig cfg, CacheManager* cache);

    void submit(int64_t id, std::vector<int32_t> prompt, int max_tokens, std::vector<int32_t> stop_ids, int priority);
    bool cancel(int64_t id);
    // A running request branches: the child takes the parent's tokens so far as its prompt, shares
    // the parent's cache pages (copy-on-write) and starts running at once, with its own limits
    // (crates/aien-scheduler/src/lib.rs:339-362).  Returns the copies the device must perform
    // (state slots).  Only between steps.
    std::vector<PageCopy> fork(int64_t parent, int64_t child, int max_tokens, std::vector<int32_t> stop_ids, int priority);
    bool has_work() const { return !waiting_.empty() || !preempted_.empty() || !running_.empty(); }
    int num_running() const { return static_cast<int>(running_.size()); }
    int num_waiting() const { return static_cast<int>(waiting_.size() + preempted_.size()); }

    // Decides the next step and allocates its cache pages.  An empty plan with has_work() true
    // means nothing can run until something finishes (or never: see take_finished for aborts).
    StepPlan plan();
    // One sampled token for every entry of the last plan that wanted logits, in entry order.
    void commit(const std::vector<int32_t>& sampled);
    // The same when the step's tokens are still on the device: every entry that wanted logits gets a
    // placeholder (-1), so that the next step can be planned (and launched, fed on the device) while
    // this one runs.  Length limits still count; a request that reaches one waits, unscheduled, for
    // its token.  resolve() later brings the values, oldest first per request: a stop id ends the
    // request there, and what it computed beyond that point is dropped.  At most one token of a
    // request may be unresolved when the next step is planned.
    void commit_deferred();
    void resolve(const std::vector<std::pair<int64_t, int32_t>>& tokens);
    // The same with the submission each value belongs to (StepEntry::arrival): a value whose request
    // ended and whose id was submitted again meanwhile is dropped instead of reaching the new request.
    void resolve_for(const std::vector<std::tuple<int64_t, int32_t, uint64_t>>& tokens);
    // The planned step failed before commit: every entry's request goes back to the cache length it
    // had (a request whose cache cannot be rewound is queued to be recomputed instead) and the step
    // counts as not planned.  Requests the plan preempted stay preempted.
    void rollback();
    // Everything the running requests hold in the cache is no longer trusted (a kernel reported a
    // broken step after later steps had been committed): each is queued to be recomputed from its
    // prompt and the tokens whose values are known; unresolved placeholders are dropped.
    void restart_running();
    std::vector<FinishEvent> take_finished();
    const SeqRecord& record(int64_t id) const { return seqs_.at(id); }
    const SchedulerMetrics& metrics() const { return metrics_; }
    const SchedulerConfig& config() const { return cfg_; }

  private:
    int min_free_pages() const;
    long long outstanding_reservation(int g) const;
    int total_pages_for(int g, int tokens, int portion) const;
    void preempt(int64_t id, StepPlan& plan);
    void finish(SeqRecord& s, FinishReason why, const std::string& msg);
    int64_t pick_victim(const std::vector<int64_t>& among) const;
    void requeue(SeqRecord& s);

    SchedulerConfig cfg_;
    CacheManager* cache_;
    std::map<int64_t, SeqRecord> seqs_;
    std::deque<int64_t> waiting_, preempted_;
    std::vector<int64_t> running_;           // kept sorted by id
    std::vector<FinishEvent> finished_;
    StepPlan last_;
    bool awaiting_commit_ = false;
    uint64_t arrivals_ = 0;
    int64_t step_counter_ = 0;
    SchedulerMetrics metrics_;
};

void bind_scheduler(pybind11::module_& m);

}  // namespace aien

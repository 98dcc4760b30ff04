#include "scheduler.h"

#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <climits>
#include <stdexcept>
#include <tuple>

namespace aien {

namespace {
inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
}  // namespace

Scheduler::Scheduler(SchedulerConfig cfg, CacheManager* cache) : cfg_(cfg), cache_(cache) {
    if (!cache_) throw std::invalid_argument("scheduler needs a cache manager");
    if (cfg_.max_batch_size <= 0 || cfg_.max_batch_tokens <= 0 || cfg_.max_prefill_tokens <= 0 ||
        cfg_.prefill_chunk_size <= 0 || cfg_.watermark_blocks < 0 || cfg_.align_step_tokens < 0)
        throw std::invalid_argument("scheduler limits must be positive");
}

void Scheduler::submit(int64_t id, std::vector<int32_t> prompt, int max_tokens, std::vector<int32_t> stop_ids, int priority) {
    if (seqs_.count(id) && seqs_[id].state != SeqState::Finished)
        throw std::invalid_argument("request " + std::to_string(id) + " is already live");
    if (prompt.empty()) throw std::invalid_argument("request " + std::to_string(id) + " has an empty prompt");
    if (max_tokens <= 0) throw std::invalid_argument("max_tokens must be positive");
    SeqRecord s;
    s.id = id;
    s.prompt = std::move(prompt);
    s.max_tokens = max_tokens;
    s.stop_ids = std::move(stop_ids);
    s.priority = priority;
    s.arrival = arrivals_++;
    const bool too_long = cfg_.max_context > 0 && static_cast<int>(s.prompt.size()) >= cfg_.max_context;
    const size_t len = s.prompt.size();
    seqs_[id] = std::move(s);
    if (too_long) {
        // never planned: its pages would outgrow the block table (the reference sizes contexts from
        // max_position_embeddings, crates/aien-inference-abi/src/model_dir.rs:116-139)
        finish(seqs_[id], FinishReason::Aborted, "prompt of " + std::to_string(len) + " tokens leaves no room below the context limit " +
               std::to_string(cfg_.max_context));
        return;
    }
    waiting_.push_back(id);
}

bool Scheduler::cancel(int64_t id) {
    auto it = seqs_.find(id);
    if (it == seqs_.end() || it->second.state == SeqState::Finished) return false;
    finish(it->second, FinishReason::Cancelled, "");
    return true;
}

std::vector<PageCopy> Scheduler::fork(int64_t parent, int64_t child, int max_tokens, std::vector<int32_t> stop_ids, int priority) {
    if (awaiting_commit_) throw std::logic_error("fork() between plan() and commit()");
    auto it = seqs_.find(parent);
    if (it == seqs_.end() || it->second.state != SeqState::Running)
        throw std::invalid_argument("request " + std::to_string(parent) + " is not running");
    if (seqs_.count(child) && seqs_[child].state != SeqState::Finished)
        throw std::invalid_argument("request " + std::to_string(child) + " is already live");
    if (max_tokens <= 0) throw std::invalid_argument("max_tokens must be positive");
    const SeqRecord& p = it->second;
    if (p.unresolved > 0) throw std::logic_error("fork() of a request whose last token is not resolved yet");
    std::vector<PageCopy> copies = cache_->fork(parent, child, p.computed);     // throws with nothing changed
    SeqRecord c;
    c.id = child;
    c.prompt = p.prompt;
    c.prompt.insert(c.prompt.end(), p.generated.begin(), p.generated.end());
    c.computed = p.computed;
    c.max_tokens = max_tokens;
    c.stop_ids = std::move(stop_ids);
    c.priority = priority;
    c.arrival = arrivals_++;
    c.state = SeqState::Running;
    seqs_[child] = std::move(c);
    running_.insert(std::upper_bound(running_.begin(), running_.end(), child), child);
    ++metrics_.admitted;
    return copies;
}

int Scheduler::min_free_pages() const {
    int m = INT_MAX;
    for (int g = 0; g < cache_->num_groups(); ++g)
        if (cache_->group(g).kind != GroupKind::State) m = std::min(m, cache_->free_count(g));
    return m;
}

int Scheduler::total_pages_for(int g, int tokens, int portion) const {
    const int ps = cache_->page_size();
    const GroupSpec& spec = cache_->group(g);
    int full = ceil_div(tokens, ps);
    if (spec.kind == GroupKind::Window) full = std::min(full, ceil_div(spec.window + portion, ps) + 1);
    return full;
}

long long Scheduler::outstanding_reservation(int g) const {
    long long total = 0;
    for (int64_t id : running_) {
        const SeqRecord& s = seqs_.at(id);
        if (!cache_->has(id)) continue;
        int held = 0;
        for (int p : cache_->table(id, g)) held += p >= 0 ? 1 : 0;
        const int want = total_pages_for(g, s.input_len() + 1, cfg_.prefill_chunk_size);
        if (want > held) total += want - held;
    }
    return total;
}

int64_t Scheduler::pick_victim(const std::vector<int64_t>& among) const {
    int64_t best = -1;
    for (int64_t id : among) {
        if (seqs_.at(id).draining) continue;             // about to end and free its pages by itself
        if (best < 0) { best = id; continue; }
        const SeqRecord& a = seqs_.at(id);
        const SeqRecord& b = seqs_.at(best);
        if (a.priority < b.priority || (a.priority == b.priority && a.arrival > b.arrival)) best = id;
    }
    return best;
}

void Scheduler::preempt(int64_t id, StepPlan& plan) {
    SeqRecord& s = seqs_.at(id);
    if (cache_->has(id)) cache_->free_request(id);
    s.computed = 0;
    s.state = SeqState::Preempted;
    ++s.preemptions;
    running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
    preempted_.push_back(id);
    plan.preempted.push_back(id);
    ++metrics_.preemptions;
}

void Scheduler::requeue(SeqRecord& s) {
    if (cache_->has(s.id)) cache_->free_request(s.id);
    while (s.unresolved > 0 && !s.generated.empty()) { s.generated.pop_back(); --s.unresolved; }
    s.unresolved = 0;
    s.draining = false;
    s.computed = 0;
    s.state = SeqState::Preempted;
    ++s.preemptions;
    running_.erase(std::remove(running_.begin(), running_.end(), s.id), running_.end());
    preempted_.push_back(s.id);
    ++metrics_.preemptions;
}

void Scheduler::rollback() {
    if (!awaiting_commit_) throw std::logic_error("rollback() without a planned step");
    awaiting_commit_ = false;
    for (const StepEntry& e : last_.entries) {
        auto it = seqs_.find(e.id);
        if (it == seqs_.end() || it->second.state != SeqState::Running || it->second.arrival != e.arrival) continue;
        SeqRecord& s = it->second;
        if (!cache_->has(e.id)) continue;
        try {
            cache_->truncate(e.id, e.start);
        } catch (const std::invalid_argument&) {
            requeue(s);                       // fixed-size state or a window that moved on: recompute
        }
    }
    --metrics_.steps;
    metrics_.tokens_scheduled -= last_.num_tokens;
    metrics_.prefill_tokens -= last_.prefill_tokens;
    metrics_.decode_tokens -= last_.num_tokens - last_.prefill_tokens;
    last_ = StepPlan{};
}

void Scheduler::restart_running() {
    if (awaiting_commit_) rollback();
    const std::vector<int64_t> ids = running_;
    for (int64_t id : ids) requeue(seqs_.at(id));
}

void Scheduler::finish(SeqRecord& s, FinishReason why, const std::string& msg) {
    if (cache_->has(s.id)) cache_->free_request(s.id);
    running_.erase(std::remove(running_.begin(), running_.end(), s.id), running_.end());
    waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), s.id), waiting_.end());
    preempted_.erase(std::remove(preempted_.begin(), preempted_.end(), s.id), preempted_.end());
    while (s.unresolved > 0 && !s.generated.empty()) { s.generated.pop_back(); --s.unresolved; }   // values that never came
    s.unresolved = 0;
    s.draining = false;
    s.state = SeqState::Finished;
    s.reason = why;
    s.message = msg;
    FinishEvent e;
    e.id = s.id;
    e.reason = why;
    e.generated = s.generated;
    e.message = msg;
    finished_.push_back(std::move(e));
    ++metrics_.finished;
}

StepPlan Scheduler::plan() {
    if (awaiting_commit_) throw std::logic_error("plan() called again before commit()");
    StepPlan p;
    p.step_id = step_counter_++;
    bool preempted_this_step = false;

    // 1. watermark: keep headroom for the running requests' next pages
    if (running_.size() > 1 && min_free_pages() < cfg_.watermark_blocks) {
        const int64_t victim = pick_victim(running_);
        if (victim >= 0) {
            preempt(victim, p);
            preempted_this_step = true;
        }
    }

    // 2. running requests in id order: one decode token, or the next portion of the input
    struct Cand { int64_t id; int n; int pending; };
    std::vector<Cand> cands;
    int seqs = 0, tokens = 0, prefill = 0;
    int held_back = 0;               // tokens taken off a portion to fill whole tiles: nobody else gets them this step
    for (int64_t id : running_) {
        if (seqs >= cfg_.max_batch_size || tokens >= cfg_.max_batch_tokens) break;
        const SeqRecord& s = seqs_.at(id);
        if (s.draining) continue;
        if (s.unresolved > 1) throw std::logic_error("plan(): request " + std::to_string(id) + " has more than one unresolved token");
        const int pending = s.input_len() - s.computed;
        int n = 1;
        if (pending > 1) {
            const int budget = std::min(cfg_.max_prefill_tokens - prefill, cfg_.max_batch_tokens - tokens);
            n = cfg_.chunk_prefill ? std::min({pending, cfg_.prefill_chunk_size, budget}) : (pending <= budget ? pending : 0);
            if (n <= 0) continue;
            prefill += n;
        }
        cands.push_back({id, n, pending});
        tokens += n;
        ++seqs;
    }
    // whole tiles: the last portion that is not the end of its input gives up what overhangs
    if (cfg_.align_step_tokens > 1) {
        for (auto it = cands.rbegin(); it != cands.rend(); ++it) {
            if (it->n <= 1 || it->n >= it->pending) continue;
            const int excess = tokens % cfg_.align_step_tokens;
            if (excess > 0 && excess * 4 <= it->n) {
                it->n -= excess;
                tokens -= excess;
                held_back += excess;
            }
            break;
        }
    }

    // 3. take the pages; when they run out, preempt the lowest-priority running request and retry
    while (!cands.empty()) {
        std::vector<std::pair<int64_t, int>> batch;
        for (const Cand& c : cands) batch.emplace_back(c.id, c.n);
        try {
            p.copies = cache_->append(batch);
            break;
        } catch (const CacheExhausted& e) {
            if (running_.size() <= 1) {
                // alone and still too large: it can never run
                SeqRecord& s = seqs_.at(cands.front().id);
                finish(s, FinishReason::Aborted, std::string(e.what()) + "; the request alone does not fit the pool");
                cands.clear();
                break;
            }
            const int64_t victim = pick_victim(running_);
            if (victim < 0) { cands.clear(); break; }     // only requests that are ending hold pages: wait for them
            for (auto it = cands.begin(); it != cands.end(); ++it)
                if (it->id == victim) { tokens -= it->n; --seqs; cands.erase(it); break; }
            preempt(victim, p);
            preempted_this_step = true;
        }
    }
    for (const Cand& c : cands) {
        const SeqRecord& s = seqs_.at(c.id);
        StepEntry e;
        e.id = c.id;
        e.arrival = s.arrival;
        e.start = s.computed;
        e.tokens.reserve(c.n);
        for (int i = 0; i < c.n; ++i) e.tokens.push_back(s.input_at(s.computed + i));
        e.wants_logits = s.computed + c.n == s.input_len();
        p.entries.push_back(std::move(e));
    }

    // 4. admission: preempted requests first, then the waiting queue, first come first served
    auto admit_from = [&](std::deque<int64_t>& q, bool was_preempted) -> bool {
        while (!q.empty()) {
            if (seqs >= cfg_.max_batch_size || tokens >= cfg_.max_batch_tokens) return false;
            const int64_t id = q.front();
            SeqRecord& s = seqs_.at(id);
            const int pending = s.input_len();
            const int budget = std::min(cfg_.max_prefill_tokens - prefill, cfg_.max_batch_tokens - tokens) - held_back;
            int n = cfg_.chunk_prefill ? std::min({pending, cfg_.prefill_chunk_size, budget})
                                       : (pending <= budget ? pending : 0);
            if (cfg_.align_step_tokens > 1 && n > 1 && n < pending) {
                const int excess = (tokens + n) % cfg_.align_step_tokens;
                if (excess > 0 && excess * 4 <= n) { n -= excess; held_back += excess; }
            }
            if (n <= 0) {
                if (!cfg_.chunk_prefill && pending > std::min(cfg_.max_prefill_tokens, cfg_.max_batch_tokens)) {
                    q.pop_front();
                    finish(s, FinishReason::Aborted, "prompt of " + std::to_string(pending) +
                           " tokens exceeds the per-step budget and chunk_prefill is off");
                    continue;
                }
                return false;
            }
            bool ok = cache_->num_requests() < cache_->max_requests();
            std::string never;
            const bool idle = running_.empty();
            for (int g = 0; g < cache_->num_groups(); ++g) {
                const GroupSpec& spec = cache_->group(g);
                if (spec.kind == GroupKind::State) {
                    if (cache_->free_count(g) < 1) ok = false;
                    continue;
                }
                const int need = total_pages_for(g, pending + 1, n);
                if (need > spec.capacity) {
                    never = std::string(kExhaustedPrefix) + " request needs " + std::to_string(need) + " pages of group " +
                            std::to_string(g) + ", the pool has " + std::to_string(spec.capacity);
                    break;
                }
                const long long avail = static_cast<long long>(cache_->free_count(g)) - outstanding_reservation(g) -
                                        ((was_preempted && !idle) ? cfg_.watermark_blocks : 0);
                if (need > avail) ok = false;
            }
            if (!never.empty()) {
                q.pop_front();
                finish(s, FinishReason::Aborted, never);
                continue;
            }
            if (!ok) return false;
            q.pop_front();
            cache_->add_request(id);
            std::vector<PageCopy> cp = cache_->append({{id, n}});
            p.copies.insert(p.copies.end(), cp.begin(), cp.end());
            s.state = SeqState::Running;
            s.computed = 0;
            running_.insert(std::upper_bound(running_.begin(), running_.end(), id), id);
            StepEntry e;
            e.id = id;
            e.arrival = s.arrival;
            e.start = 0;
            e.tokens.reserve(n);
            for (int i = 0; i < n; ++i) e.tokens.push_back(s.input_at(i));
            e.wants_logits = n == pending;
            p.entries.push_back(std::move(e));
            tokens += n;
            prefill += n;
            ++seqs;
            ++metrics_.admitted;
        }
        return true;
    };
    if (!preempted_this_step) {
        if (admit_from(preempted_, true)) admit_from(waiting_, false);
    }

    p.num_tokens = tokens;
    p.prefill_tokens = prefill;
    if (!p.entries.empty()) {
        awaiting_commit_ = true;
        ++metrics_.steps;
        metrics_.tokens_scheduled += tokens;
        metrics_.prefill_tokens += prefill;
        metrics_.decode_tokens += tokens - prefill;
    }
    last_ = p;
    return p;
}

void Scheduler::commit(const std::vector<int32_t>& sampled) {
    if (!awaiting_commit_) throw std::logic_error("commit() without a planned step");
    size_t want = 0;
    for (const StepEntry& e : last_.entries) want += e.wants_logits ? 1 : 0;
    if (sampled.size() != want)
        throw std::invalid_argument("commit: " + std::to_string(want) + " sampled tokens expected, got " + std::to_string(sampled.size()));
    awaiting_commit_ = false;
    size_t k = 0;
    for (const StepEntry& e : last_.entries) {
        const int32_t tok = e.wants_logits ? sampled[k++] : 0;
        auto it = seqs_.find(e.id);
        if (it == seqs_.end() || it->second.state != SeqState::Running || it->second.arrival != e.arrival) continue;   // cancelled meanwhile
        SeqRecord& s = it->second;
        s.computed += static_cast<int>(e.tokens.size());
        if (!e.wants_logits) continue;
        if (std::find(s.stop_ids.begin(), s.stop_ids.end(), tok) != s.stop_ids.end()) {
            finish(s, FinishReason::StopToken, "");
            continue;
        }
        s.generated.push_back(tok);
        if (static_cast<int>(s.generated.size()) >= s.max_tokens) {
            finish(s, FinishReason::LengthLimit, "");
        } else if (cfg_.max_context > 0 && s.input_len() >= cfg_.max_context) {
            finish(s, FinishReason::LengthLimit, "context limit");
        }
    }
}

void Scheduler::commit_deferred() {
    if (!awaiting_commit_) throw std::logic_error("commit_deferred() without a planned step");
    awaiting_commit_ = false;
    for (const StepEntry& e : last_.entries) {
        auto it = seqs_.find(e.id);
        if (it == seqs_.end() || it->second.state != SeqState::Running || it->second.arrival != e.arrival) continue;   // cancelled meanwhile
        SeqRecord& s = it->second;
        s.computed += static_cast<int>(e.tokens.size());
        if (!e.wants_logits) continue;
        s.generated.push_back(-1);
        ++s.unresolved;
        if (static_cast<int>(s.generated.size()) >= s.max_tokens) {
            s.draining = true;
            s.drain_message = "";
        } else if (cfg_.max_context > 0 && s.input_len() >= cfg_.max_context) {
            s.draining = true;
            s.drain_message = "context limit";
        }
    }
}

void Scheduler::resolve(const std::vector<std::pair<int64_t, int32_t>>& tokens) {
    std::vector<std::tuple<int64_t, int32_t, uint64_t>> t;
    t.reserve(tokens.size());
    for (const auto& [id, tok] : tokens) {
        auto it = seqs_.find(id);
        t.emplace_back(id, tok, it == seqs_.end() ? 0 : it->second.arrival);
    }
    resolve_for(t);
}

void Scheduler::resolve_for(const std::vector<std::tuple<int64_t, int32_t, uint64_t>>& tokens) {
    for (const auto& [id, tok, arrival] : tokens) {
        auto it = seqs_.find(id);
        if (it == seqs_.end() || it->second.state == SeqState::Finished) continue;   // ended meanwhile: the value is dropped
        if (it->second.arrival != arrival) continue;                                  // the id was submitted again: not its token
        SeqRecord& s = it->second;
        if (s.unresolved <= 0) {
            if (s.state != SeqState::Running) continue;                               // restarted meanwhile: it recomputes the token
            throw std::logic_error("resolve(): request " + std::to_string(id) + " has no unresolved token");
        }
        const size_t at = s.generated.size() - static_cast<size_t>(s.unresolved);
        if (std::find(s.stop_ids.begin(), s.stop_ids.end(), tok) != s.stop_ids.end()) {
            s.generated.resize(at);                       // the stop id is consumed; what was computed after it is dropped
            s.unresolved = 0;
            finish(s, FinishReason::StopToken, "");
            continue;
        }
        s.generated[at] = tok;
        --s.unresolved;
        if (s.draining && s.unresolved == 0) finish(s, FinishReason::LengthLimit, s.drain_message);
    }
}

std::vector<FinishEvent> Scheduler::take_finished() {
    std::vector<FinishEvent> out;
    out.swap(finished_);
    return out;
}

void bind_scheduler(pybind11::module_& m) {
    namespace py = pybind11;
    py::enum_<FinishReason>(m, "FinishReason")
        .value("NONE", FinishReason::None)
        .value("StopToken", FinishReason::StopToken)
        .value("LengthLimit", FinishReason::LengthLimit)
        .value("Cancelled", FinishReason::Cancelled)
        .value("Aborted", FinishReason::Aborted);
    py::enum_<SeqState>(m, "SeqState")
        .value("Waiting", SeqState::Waiting)
        .value("Running", SeqState::Running)
        .value("Preempted", SeqState::Preempted)
        .value("Finished", SeqState::Finished);
    py::class_<SchedulerConfig>(m, "SchedulerConfig")
        .def(py::init<>())
        .def_readwrite("max_batch_size", &SchedulerConfig::max_batch_size)
        .def_readwrite("max_batch_tokens", &SchedulerConfig::max_batch_tokens)
        .def_readwrite("max_prefill_tokens", &SchedulerConfig::max_prefill_tokens)
        .def_readwrite("prefill_chunk_size", &SchedulerConfig::prefill_chunk_size)
        .def_readwrite("chunk_prefill", &SchedulerConfig::chunk_prefill)
        .def_readwrite("watermark_blocks", &SchedulerConfig::watermark_blocks)
        .def_readwrite("max_context", &SchedulerConfig::max_context)
        .def_readwrite("align_step_tokens", &SchedulerConfig::align_step_tokens);
    py::class_<StepEntry>(m, "StepEntry")
        .def_readonly("id", &StepEntry::id)
        .def_readonly("tokens", &StepEntry::tokens)
        .def_readonly("start", &StepEntry::start)
        .def_readonly("wants_logits", &StepEntry::wants_logits)
        .def_readonly("arrival", &StepEntry::arrival);
    py::class_<StepPlan>(m, "StepPlan")
        .def_readonly("step_id", &StepPlan::step_id)
        .def_readonly("entries", &StepPlan::entries)
        .def_readonly("preempted", &StepPlan::preempted)
        .def_readonly("num_tokens", &StepPlan::num_tokens)
        .def_readonly("prefill_tokens", &StepPlan::prefill_tokens)
        .def_property_readonly("copies", [](const StepPlan& p) {
            std::vector<std::tuple<int, int, int>> out;
            for (const auto& c : p.copies) out.emplace_back(c.group, c.src, c.dst);
            return out;
        });
    py::class_<FinishEvent>(m, "FinishEvent")
        .def_readonly("id", &FinishEvent::id)
        .def_readonly("reason", &FinishEvent::reason)
        .def_readonly("generated", &FinishEvent::generated)
        .def_readonly("message", &FinishEvent::message);
    py::class_<SeqRecord>(m, "SeqRecord")
        .def_readonly("id", &SeqRecord::id)
        .def_readonly("prompt", &SeqRecord::prompt)
        .def_readonly("generated", &SeqRecord::generated)
        .def_readonly("computed", &SeqRecord::computed)
        .def_readonly("state", &SeqRecord::state)
        .def_readonly("reason", &SeqRecord::reason)
        .def_readonly("preemptions", &SeqRecord::preemptions)
        .def_readonly("unresolved", &SeqRecord::unresolved)
        .def_readonly("draining", &SeqRecord::draining)
        .def_readonly("priority", &SeqRecord::priority);
    py::class_<Scheduler>(m, "Scheduler")
        .def(py::init<SchedulerConfig, CacheManager*>(), py::arg("config"), py::arg("cache"), py::keep_alive<1, 3>())
        .def("submit", &Scheduler::submit, py::arg("id"), py::arg("prompt"), py::arg("max_tokens"),
             py::arg("stop_ids") = std::vector<int32_t>{}, py::arg("priority") = 0)
        .def("cancel", &Scheduler::cancel)
        .def("fork", [](Scheduler& s, int64_t parent, int64_t child, int max_tokens, std::vector<int32_t> stop_ids, int priority) {
                 std::vector<std::tuple<int, int, int>> out;
                 for (const auto& c : s.fork(parent, child, max_tokens, std::move(stop_ids), priority)) out.emplace_back(c.group, c.src, c.dst);
                 return out;
             }, py::arg("parent"), py::arg("child"), py::arg("max_tokens"), py::arg("stop_ids") = std::vector<int32_t>{}, py::arg("priority") = 0)
        .def("has_work", &Scheduler::has_work)
        .def_property_readonly("num_running", &Scheduler::num_running)
        .def_property_readonly("num_waiting", &Scheduler::num_waiting)
        .def("plan", &Scheduler::plan)
        .def("commit", &Scheduler::commit)
        .def("commit_deferred", &Scheduler::commit_deferred)
        .def("resolve", &Scheduler::resolve)
        .def("resolve_for", &Scheduler::resolve_for)
        .def("rollback", &Scheduler::rollback)
        .def("restart_running", &Scheduler::restart_running)
        .def("take_finished", &Scheduler::take_finished)
        .def("record", &Scheduler::record, py::return_value_policy::copy)
        .def("metrics", [](const Scheduler& s) {
            const SchedulerMetrics& x = s.metrics();
            py::dict d;
            d["steps"] = x.steps; d["tokens_scheduled"] = x.tokens_scheduled; d["prefill_tokens"] = x.prefill_tokens;
            d["decode_tokens"] = x.decode_tokens; d["preemptions"] = x.preemptions; d["finished"] = x.finished;
            d["admitted"] = x.admitted;
            return d;
        });
}

}  // namespace aien

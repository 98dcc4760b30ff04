#include "cache_manager.h"

#include <algorithm>
#include <sstream>

namespace aien {

const char* const kExhaustedPrefix = "KV pool exhausted:";

namespace {
inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
}  // namespace

CacheManager::CacheManager(int page_size, std::vector<GroupSpec> groups, int max_requests)
    : page_size_(page_size), groups_(std::move(groups)), max_requests_(max_requests) {
    if (page_size_ <= 0) throw std::invalid_argument("page_size must be positive");
    if (max_requests_ <= 0) throw std::invalid_argument("max_requests must be positive");
    free_.resize(groups_.size());
    refs_.resize(groups_.size());
    for (size_t g = 0; g < groups_.size(); ++g) {
        const GroupSpec& s = groups_[g];
        if (s.capacity < 0) throw std::invalid_argument("group capacity must not be negative");
        if (s.kind == GroupKind::Window && s.window <= 0) throw std::invalid_argument("window must be positive");
        refs_[g].assign(s.capacity, 0);
        free_[g].reserve(s.capacity);
        for (int p = s.capacity - 1; p >= 0; --p) free_[g].push_back(p);   // page 0 is handed out first
    }
    for (int r = max_requests_ - 1; r >= 0; --r) free_rows_.push_back(r);
}

const RequestEntry& CacheManager::get(int64_t id) const {
    auto it = requests_.find(id);
    if (it == requests_.end()) throw std::out_of_range("unknown request " + std::to_string(id));
    return it->second;
}
RequestEntry& CacheManager::get(int64_t id) {
    auto it = requests_.find(id);
    if (it == requests_.end()) throw std::out_of_range("unknown request " + std::to_string(id));
    return it->second;
}

std::vector<int64_t> CacheManager::request_ids() const {
    std::vector<int64_t> ids;
    ids.reserve(requests_.size());
    for (const auto& kv : requests_) ids.push_back(kv.first);
    std::sort(ids.begin(), ids.end());
    return ids;
}

int CacheManager::take_page(int g) {
    if (free_[g].empty()) {
        throw CacheExhausted(std::string(kExhaustedPrefix) + " group " + std::to_string(g) + " has no free " +
                             (groups_[g].kind == GroupKind::State ? "state slot" : "page") + " (capacity " +
                             std::to_string(groups_[g].capacity) + ")");
    }
    const int p = free_[g].back();
    free_[g].pop_back();
    refs_[g][p] = 1;
    ++metrics_.pages_allocated;
    return p;
}

void CacheManager::drop_page(int g, int page) {
    int& rc = refs_[g].at(page);
    if (rc <= 0) throw std::logic_error("page released twice");
    if (--rc == 0) {
        free_[g].push_back(page);
        ++metrics_.pages_released;
    }
}

int CacheManager::first_needed_page(int g, int next_pos) const {
    if (groups_[g].kind != GroupKind::Window) return 0;
    const int first_key = next_pos - groups_[g].window + 1;
    return first_key <= 0 ? 0 : first_key / page_size_;
}

void CacheManager::add_request(int64_t id) {
    if (has(id)) throw std::invalid_argument("request " + std::to_string(id) + " already exists");
    if (free_rows_.empty())
        throw CacheExhausted(std::string(kExhaustedPrefix) + " all " + std::to_string(max_requests_) + " request rows are in use");
    for (size_t g = 0; g < groups_.size(); ++g)
        if (groups_[g].kind == GroupKind::State && free_[g].empty())
            throw CacheExhausted(std::string(kExhaustedPrefix) + " group " + std::to_string(g) + " has no free state slot");
    RequestEntry r;
    r.id = id;
    r.row = free_rows_.back();
    free_rows_.pop_back();
    r.groups.resize(groups_.size());
    for (size_t g = 0; g < groups_.size(); ++g)
        if (groups_[g].kind == GroupKind::State) r.groups[g].state_slot = take_page(static_cast<int>(g));
    requests_.emplace(id, std::move(r));
}

std::vector<int> CacheManager::pages_needed(int64_t id, int n) const {
    std::vector<int> need(groups_.size(), 0);
    auto it = requests_.find(id);
    const RequestEntry* r = it == requests_.end() ? nullptr : &it->second;
    const int old = r ? r->num_tokens : 0;
    for (size_t g = 0; g < groups_.size(); ++g) {
        if (groups_[g].kind == GroupKind::State) {
            need[g] = r ? 0 : 1;
            continue;
        }
        if (n <= 0) continue;
        int taken = ceil_div(old + n, page_size_) - ceil_div(old, page_size_);
        int released = 0;
        if (r) {
            const GroupTable& t = r->groups[g];
            if (old % page_size_ != 0) {
                const int tail = t.pages[old / page_size_];
                if (tail >= 0 && refs_[g][tail] > 1) ++taken;                       // copy-on-write
            }
            const int fn = std::min(first_needed_page(static_cast<int>(g), old), static_cast<int>(t.pages.size()));
            for (int lp = t.first_live; lp < fn; ++lp)
                if (t.pages[lp] >= 0 && refs_[g][t.pages[lp]] == 1) ++released;
        }
        need[g] = std::max(0, taken - released);
    }
    return need;
}

bool CacheManager::can_append(const std::vector<std::pair<int64_t, int>>& batch, std::string* why) const {
    // Conservative first: pages taken, ignoring what windows give back.
    std::vector<long long> taken(groups_.size(), 0);
    for (const auto& e : batch) {
        if (!has(e.first)) {
            if (why) *why = "unknown request " + std::to_string(e.first);
            return false;
        }
        const std::vector<int> n = pages_needed(e.first, e.second);
        for (size_t g = 0; g < groups_.size(); ++g) taken[g] += n[g];
    }
    bool fits = true;
    for (size_t g = 0; g < groups_.size(); ++g)
        if (groups_[g].kind != GroupKind::State && taken[g] > static_cast<long long>(free_[g].size())) fits = false;
    if (fits) return true;
    CacheManager trial(*this);
    try {
        trial.append(batch);
        return true;
    } catch (const CacheExhausted& e) {
        if (why) *why = e.what();
        return false;
    }
}

std::vector<PageCopy> CacheManager::append(const std::vector<std::pair<int64_t, int>>& batch) {
    for (const auto& e : batch) {
        get(e.first);
        if (e.second < 0) throw std::invalid_argument("cannot append a negative number of tokens");
    }
    // Snapshot only when the batch might not fit (exact answer needs the releases applied).
    bool tight = false;
    {
        std::vector<long long> upper(groups_.size(), 0);
        for (const auto& e : batch) {
            const RequestEntry& r = get(e.first);
            for (size_t g = 0; g < groups_.size(); ++g) {
                if (groups_[g].kind == GroupKind::State) continue;
                upper[g] += ceil_div(r.num_tokens + e.second, page_size_) - ceil_div(r.num_tokens, page_size_) + 1;
            }
        }
        for (size_t g = 0; g < groups_.size(); ++g)
            if (upper[g] > static_cast<long long>(free_[g].size())) tight = true;
    }
    std::vector<std::vector<int>> free_snap, refs_snap;
    std::vector<RequestEntry> req_snap;
    CacheMetrics metrics_snap = metrics_;
    if (tight) {
        free_snap = free_;
        refs_snap = refs_;
        for (const auto& e : batch) req_snap.push_back(get(e.first));
    }
    std::vector<PageCopy> copies;
    try {
        for (const auto& e : batch) {
            RequestEntry& r = get(e.first);
            const int n = e.second;
            if (n == 0) continue;
            const int old = r.num_tokens;
            for (size_t gi = 0; gi < groups_.size(); ++gi) {
                const int g = static_cast<int>(gi);
                if (groups_[g].kind == GroupKind::State) continue;
                GroupTable& t = r.groups[g];
                // 1. give back the pages no token of this step can see any more
                const int fn = std::min(first_needed_page(g, old), static_cast<int>(t.pages.size()));
                for (int lp = t.first_live; lp < fn; ++lp) {
                    if (t.pages[lp] >= 0) {
                        drop_page(g, t.pages[lp]);
                        t.pages[lp] = -1;
                        ++metrics_.window_releases;
                    }
                }
                if (fn > t.first_live) t.first_live = fn;
                // 2. a shared, partly filled tail page is copied before it is written
                if (old % page_size_ != 0) {
                    const int lp = old / page_size_;
                    const int p = t.pages[lp];
                    if (p >= 0 && refs_[g][p] > 1) {
                        const int np = take_page(g);
                        copies.push_back(PageCopy{g, p, np});
                        drop_page(g, p);
                        t.pages[lp] = np;
                        ++metrics_.cow_copies;
                    }
                }
                // 3. new pages
                const int want = ceil_div(old + n, page_size_);
                while (static_cast<int>(t.pages.size()) < want) t.pages.push_back(take_page(g));
            }
            r.num_tokens = old + n;
        }
    } catch (const CacheExhausted&) {
        if (!tight) throw std::logic_error("cache arithmetic: an append that was predicted to fit did not");
        free_ = std::move(free_snap);
        refs_ = std::move(refs_snap);
        metrics_ = metrics_snap;
        for (auto& snap : req_snap) requests_[snap.id] = snap;
        throw;
    }
    return copies;
}

std::vector<PageCopy> CacheManager::fork(int64_t parent, int64_t child, int at_token) {
    const RequestEntry& p = get(parent);
    if (parent == child) throw std::invalid_argument("a request cannot be forked onto itself");
    if (has(child)) throw std::invalid_argument("request " + std::to_string(child) + " already exists");
    if (at_token < 0) at_token = p.num_tokens;
    if (at_token > p.num_tokens) throw std::invalid_argument("fork point lies beyond the parent's tokens");
    for (size_t g = 0; g < groups_.size(); ++g) {
        if (groups_[g].kind == GroupKind::State) {
            if (at_token != p.num_tokens)
                throw std::invalid_argument("group " + std::to_string(g) + " keeps fixed-size state: fork only at the parent's end");
        } else if (first_needed_page(static_cast<int>(g), at_token) < p.groups[g].first_live && at_token > 0) {
            throw std::invalid_argument("fork point lies before the window of group " + std::to_string(g));
        }
    }
    add_request(child);                      // may throw CacheExhausted; nothing else changed yet
    RequestEntry& c = get(child);
    const RequestEntry& pp = get(parent);    // re-fetch: the map may have rehashed
    std::vector<PageCopy> copies;
    const int np = ceil_div(at_token, page_size_);
    for (size_t gi = 0; gi < groups_.size(); ++gi) {
        const int g = static_cast<int>(gi);
        if (groups_[g].kind == GroupKind::State) {
            copies.push_back(PageCopy{g, pp.groups[g].state_slot, c.groups[g].state_slot});
            continue;
        }
        GroupTable& ct = c.groups[g];
        ct.pages.assign(pp.groups[g].pages.begin(), pp.groups[g].pages.begin() + np);
        ct.first_live = std::min(pp.groups[g].first_live, np);
        for (int page : ct.pages)
            if (page >= 0) ++refs_[g][page];
    }
    c.num_tokens = at_token;
    return copies;
}

void CacheManager::truncate(int64_t id, int num_tokens) {
    RequestEntry& r = get(id);
    if (num_tokens < 0 || num_tokens > r.num_tokens) throw std::invalid_argument("truncate: length out of range");
    if (num_tokens == r.num_tokens) return;
    for (size_t g = 0; g < groups_.size(); ++g) {
        if (groups_[g].kind == GroupKind::State)
            throw std::invalid_argument("group " + std::to_string(g) + " keeps fixed-size state and cannot be rewound");
        if (first_needed_page(static_cast<int>(g), num_tokens) < r.groups[g].first_live && num_tokens > 0)
            throw std::invalid_argument("truncate: the keys before position " + std::to_string(num_tokens) +
                                        " have left the window of group " + std::to_string(g));
    }
    const int keep = ceil_div(num_tokens, page_size_);
    for (size_t gi = 0; gi < groups_.size(); ++gi) {
        const int g = static_cast<int>(gi);
        GroupTable& t = r.groups[g];
        while (static_cast<int>(t.pages.size()) > keep) {
            if (t.pages.back() >= 0) drop_page(g, t.pages.back());
            t.pages.pop_back();
        }
        t.first_live = std::min(t.first_live, keep);
    }
    r.num_tokens = num_tokens;
}

void CacheManager::free_request(int64_t id) {
    RequestEntry& r = get(id);
    for (size_t gi = 0; gi < groups_.size(); ++gi) {
        const int g = static_cast<int>(gi);
        if (groups_[g].kind == GroupKind::State) {
            if (r.groups[g].state_slot >= 0) drop_page(g, r.groups[g].state_slot);
            continue;
        }
        // last page first: the free list is a stack, so the pages come out again in the order the
        // request held them, and a request that held a run of consecutive pages hands on a run
        // (kernels fetch consecutive pages with one copy)
        const std::vector<int>& pages = r.groups[g].pages;
        for (auto it = pages.rbegin(); it != pages.rend(); ++it)
            if (*it >= 0) drop_page(g, *it);
    }
    free_rows_.push_back(r.row);
    requests_.erase(id);
}

int CacheManager::slot_of(int64_t id, int g, int pos) const {
    const RequestEntry& r = get(id);
    if (pos < 0 || pos >= r.num_tokens) return -1;
    const int page = r.groups.at(g).pages.at(pos / page_size_);
    return page < 0 ? -1 : page * page_size_ + pos % page_size_;
}

void CacheManager::fill_meta(const std::vector<int64_t>& ids, const std::vector<int>& counts, MetaLayout& out) const {
    if (ids.size() != counts.size()) throw std::invalid_argument("fill_meta: ids and counts differ in length");
    int t = 0;
    for (size_t i = 0; i < ids.size(); ++i) {
        const RequestEntry& r = get(ids[i]);
        const int c = counts[i];
        if (c < 0 || c > r.num_tokens) throw std::invalid_argument("fill_meta: count exceeds the request's tokens");
        out.q_start[i] = t;
        out.ctx_len[i] = r.num_tokens;
        const int first = r.num_tokens - c;
        for (int j = 0; j < c; ++j) {
            out.positions[t + j] = first + j;
            out.seq_of_token[t + j] = static_cast<int32_t>(i);
        }
        for (size_t g = 0; g < groups_.size(); ++g) {
            const GroupTable& tbl = r.groups[g];
            if (groups_[g].kind == GroupKind::State) {
                if (out.slot_map[g]) out.slot_map[g][i] = tbl.state_slot;
                continue;
            }
            const int mb = out.max_blocks[g];
            if (static_cast<int>(tbl.pages.size()) > mb)
                throw std::length_error("request " + std::to_string(ids[i]) + " needs " + std::to_string(tbl.pages.size()) +
                                        " pages, block table rows hold " + std::to_string(mb));
            int32_t* row = out.block_table[g] + static_cast<size_t>(i) * mb;
            for (int b = 0; b < mb; ++b) row[b] = b < static_cast<int>(tbl.pages.size()) ? tbl.pages[b] : -1;
            for (int j = 0; j < c; ++j) {
                const int pos = first + j;
                const int page = tbl.pages[pos / page_size_];
                out.slot_map[g][t + j] = page < 0 ? -1 : page * page_size_ + pos % page_size_;
            }
        }
        t += c;
    }
    out.q_start[ids.size()] = t;
}

std::string CacheManager::check() const {
    std::ostringstream err;
    for (size_t g = 0; g < groups_.size(); ++g) {
        std::vector<int> expect(groups_[g].capacity, 0);
        for (const auto& kv : requests_) {
            const GroupTable& t = kv.second.groups[g];
            if (groups_[g].kind == GroupKind::State) {
                if (t.state_slot < 0 || t.state_slot >= groups_[g].capacity) { err << "request " << kv.first << " has no state slot in group " << g << "; "; continue; }
                ++expect[t.state_slot];
                continue;
            }
            if (static_cast<int>(t.pages.size()) != ceil_div(kv.second.num_tokens, page_size_))
                err << "request " << kv.first << " group " << g << ": table length " << t.pages.size() << " for " << kv.second.num_tokens << " tokens; ";
            for (size_t lp = 0; lp < t.pages.size(); ++lp) {
                const int p = t.pages[lp];
                if (p < 0) {
                    if (static_cast<int>(lp) >= t.first_live) err << "request " << kv.first << " group " << g << ": hole at live page " << lp << "; ";
                    continue;
                }
                if (p >= groups_[g].capacity) { err << "page id out of range; "; continue; }
                ++expect[p];
            }
        }
        std::vector<int> on_free(groups_[g].capacity, 0);
        for (int p : free_[g]) {
            if (p < 0 || p >= groups_[g].capacity) { err << "free list of group " << g << " holds bad id " << p << "; "; continue; }
            if (++on_free[p] > 1) err << "page " << p << " of group " << g << " is on the free list twice; ";
        }
        for (int p = 0; p < groups_[g].capacity; ++p) {
            if (refs_[g][p] != expect[p]) err << "page " << p << " of group " << g << ": refcount " << refs_[g][p] << ", held by " << expect[p] << " tables; ";
            if ((on_free[p] > 0) == (expect[p] > 0)) err << "page " << p << " of group " << g << (expect[p] > 0 ? " is held and free; " : " is lost (neither held nor free); ");
        }
    }
    return err.str();
}

}  // namespace aien

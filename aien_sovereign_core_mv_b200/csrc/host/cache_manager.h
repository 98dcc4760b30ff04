// Paged cache bookkeeping on the host: pages, block tables, reference counts, state slots.
//
// The manager owns no device memory.  It decides which physical page holds which logical page
// of which request, for every *group* of layers with the same needs:
//   Full    every key is kept until the request ends;
//   Window  only the last `window` keys are needed, pages the window has passed are given back;
//   State   one slot of fixed size per request (no pages).
// Each paged group has its own pool and each request one block table per group.
//
// Behaviour restated from the reference manager (crates/aien-kv-cache/src/lib.rs): LIFO free
// list that hands out page 0 first (:903-916), reference-counted pages shared by fork (:1257-1302),
// copy-on-write when appending into a shared, partly filled tail page (:1492-1556), release on
// free (:1697-1716), truncate (:1726-1778), and one authority for "how many pages would this
// append take" (:1817-1850).  Refused operations change nothing.
#pragma once
#include <cstdint>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

namespace aien {

enum class GroupKind : int { Full = 0, Window = 1, State = 2 };

struct GroupSpec {
    GroupKind kind = GroupKind::Full;
    int window = 0;      // Window groups: keys visible to a token, itself included
    int capacity = 0;    // pages (paged groups) or slots (State groups)
};

struct CacheExhausted : std::runtime_error {
    using std::runtime_error::runtime_error;
};

// Prefix of every exhaustion message; callers and tests may match on it
// (crates/aien-inference-abi/src/transformer_backend.rs:41).
extern const char* const kExhaustedPrefix;

struct PageCopy {
    int group;
    int src;
    int dst;
};

struct GroupTable {
    std::vector<int> pages;   // logical page index -> physical page, -1 once released
    int first_live = 0;       // logical pages below this index were released (Window groups)
    int state_slot = -1;      // State groups
};

struct RequestEntry {
    int64_t id = 0;
    int num_tokens = 0;
    int row = -1;             // stable small index while the request lives
    std::vector<GroupTable> groups;
};

struct CacheMetrics {
    long long cow_copies = 0;
    long long pages_allocated = 0;
    long long pages_released = 0;
    long long window_releases = 0;
};

class CacheManager {
  public:
    CacheManager(int page_size, std::vector<GroupSpec> groups, int max_requests);

    int page_size() const { return page_size_; }
    int num_groups() const { return static_cast<int>(groups_.size()); }
    const GroupSpec& group(int g) const { return groups_.at(g); }
    int max_requests() const { return max_requests_; }
    int num_requests() const { return static_cast<int>(requests_.size()); }
    bool has(int64_t id) const { return requests_.count(id) != 0; }
    int num_tokens(int64_t id) const { return get(id).num_tokens; }
    int row_of(int64_t id) const { return get(id).row; }
    int free_count(int g) const { return static_cast<int>(free_[g].size()); }
    int refcount(int g, int page) const { return refs_.at(g).at(page); }
    const CacheMetrics& metrics() const { return metrics_; }
    std::vector<int64_t> request_ids() const;

    // Registers a request with no tokens; takes a state slot in every State group.
    void add_request(int64_t id);
    // Pages (per group) that append(id, n) would take from the free lists, after the pages it
    // gives back first.  `id` may be unknown (a request about to be added): then from empty.
    std::vector<int> pages_needed(int64_t id, int n) const;
    // Whether every (id, n) of a batch can be appended together.
    bool can_append(const std::vector<std::pair<int64_t, int>>& batch, std::string* why = nullptr) const;
    // Makes room for n more tokens of every request in the batch and advances their lengths.
    // All or nothing: throws CacheExhausted with nothing changed.  Returns the page copies the
    // device must perform (copy-on-write) before the step writes.
    std::vector<PageCopy> append(const std::vector<std::pair<int64_t, int>>& batch);
    // child shares the parent's first `at_token` tokens (at_token < 0: all of them).
    std::vector<PageCopy> fork(int64_t parent, int64_t child, int at_token);
    void truncate(int64_t id, int num_tokens);
    void free_request(int64_t id);

    // Physical token slot (page * page_size + offset) of position `pos`; -1 if released/absent.
    int slot_of(int64_t id, int g, int pos) const;
    int state_slot(int64_t id, int g) const { return get(id).groups.at(g).state_slot; }
    const std::vector<int>& table(int64_t id, int g) const { return get(id).groups.at(g).pages; }

    // Writes positions, row mapping, block tables and slot maps of a step that brings `counts[i]`
    // new tokens of `ids[i]` (already appended) into int32 arrays.  Returns false if a table is
    // longer than max_blocks.
    struct MetaLayout {
        int32_t* positions;     // [T]
        int32_t* seq_of_token;  // [T]
        int32_t* q_start;       // [S+1]
        int32_t* ctx_len;       // [S]
        std::vector<int32_t*> block_table;  // per group [S * max_blocks] (nullptr for State)
        std::vector<int32_t*> slot_map;     // per group [T] (State: [S] state slots)
        std::vector<int> max_blocks;        // per group
    };
    void fill_meta(const std::vector<int64_t>& ids, const std::vector<int>& counts, MetaLayout& out) const;

    // Invariants: every page is free xor referenced; refcounts equal the number of tables
    // holding the page; no page twice on the free list.  Returns "" or what is wrong.
    std::string check() const;

  private:
    const RequestEntry& get(int64_t id) const;
    RequestEntry& get(int64_t id);
    int take_page(int g);
    void drop_page(int g, int page);
    // first logical page still needed by a request whose next token sits at position `next_pos`
    int first_needed_page(int g, int next_pos) const;

    int page_size_;
    std::vector<GroupSpec> groups_;
    int max_requests_;
    std::vector<std::vector<int>> free_;     // per group LIFO
    std::vector<std::vector<int>> refs_;     // per group per page/slot
    std::unordered_map<int64_t, RequestEntry> requests_;
    std::vector<int> free_rows_;
    CacheMetrics metrics_;
};

}  // namespace aien

// Host runtime of phaseshift_b200: request/sequence bookkeeping that must make identical decisions on
// every tensor-parallel rank and that is unit-testable without a GPU.
//
//   SlotPool / PagePool / SequenceState  -- sequence slots with generation counters (stale-handle
//       detection), KV page free list, two-phase append (reserve -> commit | rollback) and poisoning
//       (reference: models/qwen35/state/{sequence_slot_pool,paged_kv_pool,paged_sequence_state}.h)
//   KvBanker                             -- Banker's-algorithm admission and page grants, so a set of
//       admitted requests can always run to completion (reference: runtime/kv_banker.cpp:19-110)
//   Scheduler                            -- token-budget step planner: decodes first, then prefill
//       chunks, cut at prefix-cache checkpoints (reference: runtime/token_budget_scheduler.cpp:10-141)
//   Batcher                              -- continuous batching state machine: queue, admit, plan,
//       commit sampled tokens, finish (eos / length / cancelled / error)
//       (reference: runtime/continuous_batcher.cpp:105-560)
//   PrefixIndex                          -- exact-token prefix lookup with LRU eviction
//       (reference: runtime/prefix_cache.cpp, docs/developer/prefix_cache.md:123-140)
//   spec_greedy_accept / SpecTransaction / NgramTail -- speculative decoding helpers
//       (reference: runtime/spec_decode.h:14-147, runtime/ngram_tail.cpp)
#pragma once

#include <cstdint>
#include <deque>
#include <list>
#include <map>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace psrt {

enum class StatusCode : int {
    ok = 0, invalid_argument, out_of_range, unsupported, resource_exhausted, stale_handle, poisoned,
    cuda_error, nccl_error, io_error, format_error, timeout, internal
};
const char* status_name(StatusCode c);

struct Error : std::runtime_error {
    StatusCode code;
    Error(StatusCode c, const std::string& m) : std::runtime_error(std::string(status_name(c)) + ": " + m), code(c) {}
};

// Overflow-checked size arithmetic (reference: include/phaseshift/core/status.h:151-211).
uint64_t checked_add(uint64_t a, uint64_t b);
uint64_t checked_mul(uint64_t a, uint64_t b);
uint64_t align_up(uint64_t v, uint64_t a);

// ------------------------------------------------------------------------------------------------ pools
struct Handle { int32_t slot = -1; uint32_t generation = 0; };

class SlotPool {
public:
    explicit SlotPool(uint32_t max_slots);
    Handle acquire();                       // slot = -1 when exhausted
    void release(Handle h);                 // throws stale_handle
    bool valid(Handle h) const;
    uint32_t free_count() const { return (uint32_t)free_.size(); }
    uint32_t capacity() const { return (uint32_t)generation_.size(); }
private:
    std::vector<uint32_t> generation_;
    std::vector<int32_t> free_;
    std::vector<uint8_t> live_;
};

class PagePool {
public:
    explicit PagePool(uint32_t num_pages);  // page 0 is reserved (never handed out)
    int32_t acquire();                      // -1 when exhausted
    void release(int32_t page);
    uint32_t free_count() const { return (uint32_t)free_.size(); }
    uint32_t capacity() const { return capacity_; }
private:
    uint32_t capacity_;
    std::vector<int32_t> free_;
    std::vector<uint8_t> used_;
};

struct BlockUpdate { int32_t slot; uint32_t block; int32_t page; };   // device block-table write

class SequenceState {
public:
    Handle handle;
    uint32_t position = 0;                  // committed tokens
    uint32_t max_seq_len = 0;
    bool poisoned = false;
    std::vector<int32_t> pages;             // block table
    // reserve pages so positions < new_end are mapped; appends the device updates to `out`
    void reserve(uint32_t new_end, uint32_t page_tokens, PagePool& pool, std::vector<BlockUpdate>& out);
    void commit(uint32_t new_end);
    void rollback(uint32_t page_tokens, PagePool& pool, std::vector<BlockUpdate>& out);   // drop pages past `position`
    void trim_to(uint32_t new_position, uint32_t page_tokens, PagePool& pool, std::vector<BlockUpdate>& out);
    void release_all(PagePool& pool);
    uint32_t reserved_before_ = 0;
};

uint32_t pages_for(uint32_t tokens, uint32_t page_tokens);
uint32_t additional_pages(uint32_t position, uint32_t have_pages, uint32_t add_tokens, uint32_t page_tokens);

// ------------------------------------------------------------------------------------------------ banker
struct BankerProcess { uint32_t allocated = 0; uint32_t max_claim = 0; };

class KvBanker {
public:
    uint32_t available = 0;
    std::vector<BankerProcess> processes;
    bool is_safe() const;
    bool can_admit(uint32_t max_claim) const;                 // would adding a process keep the state safe?
    uint32_t max_safe_grant(size_t idx, uint32_t want) const; // largest g <= want keeping the state safe
};

// ------------------------------------------------------------------------------------------------ requests
enum class RequestState : int { Queued = 0, Active = 1, Finished = 2 };
enum class FinishReason : int { None = 0, Eos = 1, Length = 2, Cancelled = 3, Error = 4 };
const char* finish_name(FinishReason r);    // stop / length / cancelled / error / none

struct Sampling { float temperature = 0.f; float top_p = 1.f; uint32_t top_k = 0; uint64_t seed = 0; };

struct Request {
    uint64_t id = 0;
    std::vector<int32_t> prompt;
    std::vector<int32_t> generated;
    uint32_t max_new_tokens = 0;
    Sampling sampling;
    std::vector<int32_t> stop_tokens;
    uint32_t checkpoint_position = 0;       // prefix-cache boundary inside the prompt (0 = none)
    bool checkpoint_saved = false;
    uint32_t restored_tokens = 0;           // prefix-cache hit length
    RequestState state = RequestState::Queued;
    FinishReason finish = FinishReason::None;
    SequenceState seq;
    int32_t pending_token = -1;             // sampled, not yet fed back
    uint32_t prefill_tokens = 0;            // prompt tokens actually computed
    std::string error;
};

struct PlannedSeq {
    uint64_t request_id; int32_t slot; uint32_t pos_start; uint32_t token_offset; uint32_t n_tokens;
    bool sample; bool is_decode; uint32_t sample_index;
};
struct StepPlan {
    std::vector<PlannedSeq> seqs;
    std::vector<int32_t> tokens;
    std::vector<BlockUpdate> block_updates;
    uint32_t n_sampled = 0;
    bool empty() const { return seqs.empty(); }
};

struct Event { int kind; uint64_t request_id; int32_t token; };   // kind 0 = token, 1 = done, 2 = error

struct BatcherConfig {
    uint32_t max_slots = 4, num_pages = 0, page_tokens = 16, max_seq_len = 512;
    uint32_t max_step_tokens = 2048, max_step_requests = 0;
    bool full_claim = false;                // ConservativeFullClaim: reserve a request's worst case at admission
};

class Batcher {
public:
    explicit Batcher(const BatcherConfig& cfg);
    uint64_t submit(std::vector<int32_t> prompt, uint32_t max_new_tokens, Sampling s, std::vector<int32_t> stop_tokens,
                    uint32_t checkpoint_position);
    bool cancel(uint64_t id);
    void cancel_all();
    // admission (returns ids admitted this call, in order; the caller resets device state / restores prefixes)
    std::vector<uint64_t> admit();
    // mark `n` prompt tokens as already present in the sequence (prefix-cache restore), pages reserved here
    void restore_prefix(uint64_t id, uint32_t n_tokens, std::vector<BlockUpdate>& updates);
    StepPlan plan();
    // commit a finished step: `sampled` holds one token per sampled sequence in plan order
    std::vector<Event> commit(const StepPlan& plan, const std::vector<int32_t>& sampled);
    // the step failed on the device: roll reservations back and finish the involved requests with Error
    std::vector<Event> fail(const StepPlan& plan, const std::string& why);
    const Request* find(uint64_t id) const;
    Request* find_mut(uint64_t id);
    void retire(uint64_t id);               // drop a finished request
    uint32_t active_count() const;
    uint32_t queued_count() const;
    uint32_t free_pages() const { return pages_.free_count(); }
    bool idle() const;
    std::vector<BlockUpdate> take_release_updates();   // block-table clears produced by finished requests
    KvBanker banker_snapshot() const;
    BatcherConfig cfg;
private:
    void finish(Request& r, FinishReason why, std::vector<Event>& ev);
    uint32_t worst_case_pages(const Request& r) const;
    SlotPool slots_;
    PagePool pages_;
    std::list<Request> requests_;
    std::unordered_map<uint64_t, std::list<Request>::iterator> index_;
    std::vector<BlockUpdate> release_updates_;
    uint64_t next_id_ = 1;
};

// ------------------------------------------------------------------------------------------------ prefix cache index
struct PrefixHit { int64_t entry = -1; uint32_t tokens = 0; };

class PrefixIndex {
public:
    PrefixIndex(uint32_t max_entries, uint32_t capacity_tokens, uint32_t min_tokens);
    // longest stored sequence that is a strict prefix of `prompt` (exact token comparison)
    PrefixHit lookup(const std::vector<int32_t>& prompt);
    // returns the entry id to fill (evicting LRU entries as needed; evicted ids are appended to `evicted`),
    // or -1 for a benign skip (too short / too long / already present)
    int64_t insert(const std::vector<int32_t>& tokens, std::vector<int64_t>& evicted);
    void erase(int64_t entry);
    uint32_t used_tokens() const { return used_; }
    uint32_t entries() const { return (uint32_t)entries_.size(); }
    uint64_t hits = 0, misses = 0, inserts = 0, evictions = 0, skipped = 0;
private:
    struct Entry { int64_t id; std::vector<int32_t> tokens; };
    std::list<Entry> entries_;              // front = most recently used
    uint32_t max_entries_, capacity_, min_tokens_, used_ = 0;
    int64_t next_id_ = 0;
};

// ------------------------------------------------------------------------------------------------ speculative decoding
struct AcceptResult { uint32_t accepted; int32_t next_token; bool full; };
// drafts[i] was fed at row i+1; target[i] is the target's sample at row i (row 0 = the anchor token).
// Longest prefix with drafts[i] == target[i]; next_token = target[accepted] (correction, or bonus on full accept).
AcceptResult spec_greedy_accept(const std::vector<int32_t>& drafts, const std::vector<int32_t>& target);

class SpecTransaction {   // Idle -> Proposed -> Verified -> (Committed | RolledBack) -> Idle
public:
    enum State { Idle = 0, Proposed, Verified, Committed, RolledBack };
    State state = Idle;
    uint32_t base_position = 0, rows = 0, accepted = 0;
    void begin(uint32_t position, uint32_t n_rows);
    void verified(uint32_t n_accepted);
    uint32_t commit();        // new position
    void rollback();
    void reset();
};

// n-gram continuation: find the latest earlier occurrence of the last `n` tokens and propose what followed.
std::vector<int32_t> ngram_tail(const std::vector<int32_t>& history, uint32_t n, uint32_t max_tokens);

// ------------------------------------------------------------------------------------------------ misc
uint32_t crc32(const uint8_t* data, size_t n, uint32_t seed = 0);

}  // namespace psrt

// Pools, KV banker, scheduler + continuous batcher, prefix index, speculative helpers (see ps_runtime.h).
#include "ps_runtime.h"

#include <algorithm>
#include <limits>

namespace psrt {

const char* status_name(StatusCode c) {
    switch (c) {
        case StatusCode::ok: return "ok";
        case StatusCode::invalid_argument: return "invalid_argument";
        case StatusCode::out_of_range: return "out_of_range";
        case StatusCode::unsupported: return "unsupported";
        case StatusCode::resource_exhausted: return "resource_exhausted";
        case StatusCode::stale_handle: return "stale_handle";
        case StatusCode::poisoned: return "poisoned";
        case StatusCode::cuda_error: return "cuda_error";
        case StatusCode::nccl_error: return "nccl_error";
        case StatusCode::io_error: return "io_error";
        case StatusCode::format_error: return "format_error";
        case StatusCode::timeout: return "timeout";
        case StatusCode::internal: return "internal";
    }
    return "unknown";
}

uint64_t checked_add(uint64_t a, uint64_t b) {
    if (a > std::numeric_limits<uint64_t>::max() - b) throw Error(StatusCode::out_of_range, "size overflow in add");
    return a + b;
}
uint64_t checked_mul(uint64_t a, uint64_t b) {
    if (a != 0 && b > std::numeric_limits<uint64_t>::max() / a) throw Error(StatusCode::out_of_range, "size overflow in mul");
    return a * b;
}
uint64_t align_up(uint64_t v, uint64_t a) {
    if (a == 0) throw Error(StatusCode::invalid_argument, "alignment 0");
    return checked_add(v, a - 1) / a * a;
}

// ------------------------------------------------------------------------------------------------ pools
SlotPool::SlotPool(uint32_t max_slots) : generation_(max_slots, 0), live_(max_slots, 0) {
    for (int32_t s = (int32_t)max_slots - 1; s >= 0; --s) free_.push_back(s);
}
Handle SlotPool::acquire() {
    Handle h;
    if (free_.empty()) return h;
    h.slot = free_.back();
    free_.pop_back();
    h.generation = generation_[h.slot];
    live_[h.slot] = 1;
    return h;
}
bool SlotPool::valid(Handle h) const {
    return h.slot >= 0 && (size_t)h.slot < generation_.size() && live_[h.slot] && generation_[h.slot] == h.generation;
}
void SlotPool::release(Handle h) {
    if (!valid(h)) throw Error(StatusCode::stale_handle, "sequence handle is stale or was never acquired");
    live_[h.slot] = 0;
    ++generation_[h.slot];
    free_.push_back(h.slot);
}

PagePool::PagePool(uint32_t num_pages) : capacity_(num_pages), used_(num_pages, 0) {
    for (int32_t p = (int32_t)num_pages - 1; p >= 1; --p) free_.push_back(p);
}
int32_t PagePool::acquire() {
    if (free_.empty()) return -1;
    const int32_t p = free_.back();
    free_.pop_back();
    used_[p] = 1;
    return p;
}
void PagePool::release(int32_t page) {
    if (page <= 0 || (uint32_t)page >= capacity_ || !used_[page]) throw Error(StatusCode::invalid_argument, "bad page release");
    used_[page] = 0;
    free_.push_back(page);
}

uint32_t pages_for(uint32_t tokens, uint32_t page_tokens) { return (tokens + page_tokens - 1) / page_tokens; }
uint32_t additional_pages(uint32_t position, uint32_t have_pages, uint32_t add_tokens, uint32_t page_tokens) {
    const uint32_t need = pages_for(position + add_tokens, page_tokens);
    return need > have_pages ? need - have_pages : 0;
}

void SequenceState::reserve(uint32_t new_end, uint32_t page_tokens, PagePool& pool, std::vector<BlockUpdate>& out) {
    if (poisoned) throw Error(StatusCode::poisoned, "sequence is poisoned");
    if (new_end > max_seq_len) throw Error(StatusCode::out_of_range, "append exceeds max_seq_len");
    const uint32_t need = pages_for(new_end, page_tokens);
    reserved_before_ = (uint32_t)pages.size();
    while (pages.size() < need) {
        const int32_t p = pool.acquire();
        if (p < 0) {
            rollback(page_tokens, pool, out);
            throw Error(StatusCode::resource_exhausted, "out of KV pages");
        }
        out.push_back({handle.slot, (uint32_t)pages.size(), p});
        pages.push_back(p);
    }
}
void SequenceState::commit(uint32_t new_end) {
    if (new_end < position) throw Error(StatusCode::invalid_argument, "commit moves backwards");
    position = new_end;
}
void SequenceState::trim_to(uint32_t new_position, uint32_t page_tokens, PagePool& pool, std::vector<BlockUpdate>& out) {
    const uint32_t keep = pages_for(new_position == 0 ? 0 : new_position, page_tokens);
    while (pages.size() > keep) {
        pool.release(pages.back());
        pages.pop_back();
        out.push_back({handle.slot, (uint32_t)pages.size(), -1});
    }
    if (new_position < position) position = new_position;
}
void SequenceState::rollback(uint32_t page_tokens, PagePool& pool, std::vector<BlockUpdate>& out) {
    const uint32_t keep = std::max(pages_for(position, page_tokens), std::min<uint32_t>(reserved_before_, (uint32_t)pages.size()));
    while (pages.size() > keep) {
        pool.release(pages.back());
        pages.pop_back();
        out.push_back({handle.slot, (uint32_t)pages.size(), -1});
    }
}
void SequenceState::release_all(PagePool& pool) {
    for (int32_t p : pages) pool.release(p);
    pages.clear();
}

// ------------------------------------------------------------------------------------------------ banker
bool KvBanker::is_safe() const {
    // classic safety check: repeatedly finish any process whose remaining need fits in `work`
    std::vector<uint8_t> done(processes.size(), 0);
    uint64_t work = available;
    size_t left = processes.size();
    bool progress = true;
    while (left > 0 && progress) {
        progress = false;
        for (size_t i = 0; i < processes.size(); ++i) {
            if (done[i]) continue;
            const auto& p = processes[i];
            const uint32_t need = p.max_claim > p.allocated ? p.max_claim - p.allocated : 0;
            if (need <= work) {
                work += p.allocated;
                done[i] = 1;
                --left;
                progress = true;
            }
        }
    }
    return left == 0;
}
bool KvBanker::can_admit(uint32_t max_claim) const {
    KvBanker t = *this;
    t.processes.push_back({0, max_claim});
    return t.is_safe();
}
uint32_t KvBanker::max_safe_grant(size_t idx, uint32_t want) const {
    if (idx >= processes.size()) return 0;
    const auto& p = processes[idx];
    const uint32_t room = p.max_claim > p.allocated ? p.max_claim - p.allocated : 0;
    uint32_t hi = std::min({want, room, available});
    uint32_t lo = 0;    // grant of 0 keeps the current (safe) state
    auto safe_with = [&](uint32_t g) {
        KvBanker t = *this;
        t.available -= g;
        t.processes[idx].allocated += g;
        return t.is_safe();
    };
    if (hi == 0) return 0;
    if (safe_with(hi)) return hi;
    while (lo + 1 < hi) {   // safety is monotone in g for a single process
        const uint32_t mid = lo + (hi - lo) / 2;
        if (safe_with(mid)) lo = mid; else hi = mid;
    }
    return lo;
}

// ------------------------------------------------------------------------------------------------ batcher
const char* finish_name(FinishReason r) {
    switch (r) {
        case FinishReason::Eos: return "stop";
        case FinishReason::Length: return "length";
        case FinishReason::Cancelled: return "cancelled";
        case FinishReason::Error: return "error";
        default: return "none";
    }
}

Batcher::Batcher(const BatcherConfig& c) : cfg(c), slots_(c.max_slots), pages_(c.num_pages) {
    if (c.page_tokens == 0 || c.max_slots == 0 || c.num_pages < 2) throw Error(StatusCode::invalid_argument, "bad batcher config");
}

uint64_t Batcher::submit(std::vector<int32_t> prompt, uint32_t max_new_tokens, Sampling s, std::vector<int32_t> stop_tokens,
                         uint32_t checkpoint_position) {
    if (prompt.empty()) throw Error(StatusCode::invalid_argument, "empty prompt");
    if (prompt.size() + max_new_tokens > cfg.max_seq_len)
        throw Error(StatusCode::out_of_range, "prompt + max_new_tokens exceeds max_seq_len");
    if (checkpoint_position >= prompt.size()) checkpoint_position = 0;
    Request r;
    r.id = next_id_++;
    r.prompt = std::move(prompt);
    r.max_new_tokens = max_new_tokens;
    r.sampling = s;
    r.stop_tokens = std::move(stop_tokens);
    r.checkpoint_position = checkpoint_position;
    r.seq.max_seq_len = cfg.max_seq_len;
    requests_.push_back(std::move(r));
    index_[requests_.back().id] = std::prev(requests_.end());
    return requests_.back().id;
}

uint32_t Batcher::worst_case_pages(const Request& r) const {
    return pages_for((uint32_t)r.prompt.size() + r.max_new_tokens, cfg.page_tokens);
}

KvBanker Batcher::banker_snapshot() const {
    KvBanker b;
    b.available = pages_.free_count();
    for (const auto& r : requests_)
        if (r.state == RequestState::Active) b.processes.push_back({(uint32_t)r.seq.pages.size(), worst_case_pages(r)});
    return b;
}

std::vector<uint64_t> Batcher::admit() {
    std::vector<uint64_t> out;
    for (auto& r : requests_) {
        if (r.state != RequestState::Queued) continue;
        if (slots_.free_count() == 0) break;
        KvBanker b = banker_snapshot();
        const uint32_t claim = worst_case_pages(r);
        if (claim > pages_.capacity() - 1) {   // can never run
            std::vector<Event> ev;
            r.error = "request needs more KV pages than the pool holds";
            r.state = RequestState::Finished; r.finish = FinishReason::Error;
            continue;
        }
        if (cfg.full_claim) {
            uint64_t committed = 0;
            for (const auto& p : b.processes) committed += p.max_claim;
            if (committed + claim > pages_.capacity() - 1) break;
        } else if (!b.can_admit(claim)) {
            break;      // FIFO: do not let later requests overtake
        }
        r.seq.handle = slots_.acquire();
        r.state = RequestState::Active;
        out.push_back(r.id);
    }
    return out;
}

void Batcher::restore_prefix(uint64_t id, uint32_t n_tokens, std::vector<BlockUpdate>& updates) {
    Request* r = find_mut(id);
    if (r == nullptr || r->state != RequestState::Active) throw Error(StatusCode::invalid_argument, "restore on inactive request");
    if (n_tokens >= r->prompt.size() || r->seq.position != 0) throw Error(StatusCode::invalid_argument, "bad prefix restore length");
    r->seq.reserve(n_tokens, cfg.page_tokens, pages_, updates);
    r->seq.commit(n_tokens);
    r->restored_tokens = n_tokens;
    if (r->checkpoint_position != 0 && n_tokens >= r->checkpoint_position) r->checkpoint_saved = true;
}

StepPlan Batcher::plan() {
    StepPlan plan;
    KvBanker bank = banker_snapshot();
    auto budget_left = [&]() { return cfg.max_step_tokens - (uint32_t)plan.tokens.size(); };
    auto cap_reached = [&]() { return cfg.max_step_requests != 0 && plan.seqs.size() >= cfg.max_step_requests; };
    // pass 1: decodes (one token each), pass 2: prefill chunks
    for (int pass = 0; pass < 2; ++pass) {
        size_t proc = 0;
        for (auto& r : requests_) {
            if (r.state != RequestState::Active) continue;
            const size_t pi = proc++;
            const uint32_t pos = r.seq.position;
            const bool in_prefill = pos < r.prompt.size();
            if ((pass == 0) == in_prefill) continue;
            if (budget_left() < 1 || cap_reached()) break;
            uint32_t take;
            if (pass == 0) {
                if (r.pending_token < 0) continue;
                take = 1;
                const uint32_t delta = additional_pages(pos, (uint32_t)r.seq.pages.size(), 1, cfg.page_tokens);
                if (delta > 0 && bank.max_safe_grant(pi, delta) < delta) continue;
            } else {
                take = std::min<uint32_t>((uint32_t)r.prompt.size() - pos, budget_left());
                const uint32_t want = additional_pages(pos, (uint32_t)r.seq.pages.size(), take, cfg.page_tokens);
                if (want > 0) {
                    const uint32_t safe = bank.max_safe_grant(pi, want);
                    if (safe == 0) continue;
                    const uint64_t max_end = (uint64_t)(r.seq.pages.size() + safe) * cfg.page_tokens;
                    if (max_end <= pos) continue;
                    take = (uint32_t)std::min<uint64_t>(take, max_end - pos);
                }
                // stop exactly at the prefix-cache boundary so cached and uncached runs chunk identically
                if (r.checkpoint_position > 0 && !r.checkpoint_saved && pos < r.checkpoint_position &&
                    take > r.checkpoint_position - pos)
                    take = r.checkpoint_position - pos;
            }
            const uint32_t before = (uint32_t)r.seq.pages.size();
            try {
                r.seq.reserve(pos + take, cfg.page_tokens, pages_, plan.block_updates);
            } catch (const Error&) {
                continue;
            }
            const uint32_t granted = (uint32_t)r.seq.pages.size() - before;
            bank.available -= granted;
            bank.processes[pi].allocated += granted;
            PlannedSeq ps;
            ps.request_id = r.id; ps.slot = r.seq.handle.slot; ps.pos_start = pos;
            ps.token_offset = (uint32_t)plan.tokens.size(); ps.n_tokens = take; ps.is_decode = pass == 0;
            ps.sample_index = (uint32_t)r.generated.size();
            if (pass == 0) {
                plan.tokens.push_back(r.pending_token);
                ps.sample = true;
            } else {
                plan.tokens.insert(plan.tokens.end(), r.prompt.begin() + pos, r.prompt.begin() + pos + take);
                ps.sample = (pos + take == r.prompt.size()) && r.max_new_tokens > 0;
            }
            if (ps.sample) ++plan.n_sampled;
            plan.seqs.push_back(ps);
        }
    }
    return plan;
}

void Batcher::finish(Request& r, FinishReason why, std::vector<Event>& ev) {
    if (r.state == RequestState::Finished) return;
    if (r.state == RequestState::Active) {
        for (uint32_t b = 0; b < r.seq.pages.size(); ++b) release_updates_.push_back({r.seq.handle.slot, b, -1});
        r.seq.release_all(pages_);
        slots_.release(r.seq.handle);
    }
    r.state = RequestState::Finished;
    r.finish = why;
    r.pending_token = -1;
    ev.push_back({why == FinishReason::Error ? 2 : 1, r.id, -1});
}

std::vector<Event> Batcher::commit(const StepPlan& plan, const std::vector<int32_t>& sampled) {
    if (sampled.size() != plan.n_sampled) throw Error(StatusCode::invalid_argument, "sampled token count does not match the plan");
    std::vector<Event> ev;
    size_t si = 0;
    for (const auto& ps : plan.seqs) {
        Request* r = find_mut(ps.request_id);
        const int32_t tok = ps.sample ? sampled[si++] : -1;
        if (r == nullptr || r->state != RequestState::Active) continue;   // cancelled while in flight
        r->seq.commit(ps.pos_start + ps.n_tokens);
        if (!ps.is_decode) {
            r->prefill_tokens += ps.n_tokens;
            if (r->checkpoint_position != 0 && r->seq.position >= r->checkpoint_position) r->checkpoint_saved = true;
        }
        if (!ps.sample) continue;
        if (tok < 0) { r->error = "sampling failed"; finish(*r, FinishReason::Error, ev); continue; }
        r->generated.push_back(tok);
        ev.push_back({0, r->id, tok});
        const bool is_stop = std::find(r->stop_tokens.begin(), r->stop_tokens.end(), tok) != r->stop_tokens.end();
        if (is_stop) finish(*r, FinishReason::Eos, ev);
        else if (r->generated.size() >= r->max_new_tokens) finish(*r, FinishReason::Length, ev);
        else r->pending_token = tok;
    }
    // prompts with max_new_tokens == 0 finish once prefilled
    for (auto& r : requests_)
        if (r.state == RequestState::Active && r.max_new_tokens == 0 && r.seq.position >= r.prompt.size())
            finish(r, FinishReason::Length, ev);
    return ev;
}

std::vector<Event> Batcher::fail(const StepPlan& plan, const std::string& why) {
    std::vector<Event> ev;
    for (const auto& ps : plan.seqs) {
        Request* r = find_mut(ps.request_id);
        if (r == nullptr || r->state != RequestState::Active) continue;
        r->seq.poisoned = true;
        r->error = why;
        finish(*r, FinishReason::Error, ev);
    }
    return ev;
}

bool Batcher::cancel(uint64_t id) {
    Request* r = find_mut(id);
    if (r == nullptr || r->state == RequestState::Finished) return false;
    std::vector<Event> ev;
    finish(*r, FinishReason::Cancelled, ev);
    return true;
}
void Batcher::cancel_all() {
    std::vector<Event> ev;
    for (auto& r : requests_) finish(r, FinishReason::Cancelled, ev);
}
const Request* Batcher::find(uint64_t id) const {
    auto it = index_.find(id);
    return it == index_.end() ? nullptr : &*it->second;
}
Request* Batcher::find_mut(uint64_t id) {
    auto it = index_.find(id);
    return it == index_.end() ? nullptr : &*it->second;
}
void Batcher::retire(uint64_t id) {
    auto it = index_.find(id);
    if (it == index_.end()) return;
    if (it->second->state != RequestState::Finished) throw Error(StatusCode::invalid_argument, "retire of a live request");
    requests_.erase(it->second);
    index_.erase(it);
}
uint32_t Batcher::active_count() const {
    uint32_t n = 0;
    for (const auto& r : requests_) n += r.state == RequestState::Active;
    return n;
}
uint32_t Batcher::queued_count() const {
    uint32_t n = 0;
    for (const auto& r : requests_) n += r.state == RequestState::Queued;
    return n;
}
bool Batcher::idle() const { return active_count() == 0 && queued_count() == 0; }
std::vector<BlockUpdate> Batcher::take_release_updates() {
    std::vector<BlockUpdate> out;
    out.swap(release_updates_);
    return out;
}

// ------------------------------------------------------------------------------------------------ prefix index
PrefixIndex::PrefixIndex(uint32_t max_entries, uint32_t capacity_tokens, uint32_t min_tokens)
    : max_entries_(max_entries), capacity_(capacity_tokens), min_tokens_(min_tokens) {}

PrefixHit PrefixIndex::lookup(const std::vector<int32_t>& prompt) {
    auto best = entries_.end();
    for (auto it = entries_.begin(); it != entries_.end(); ++it) {
        const auto& t = it->tokens;
        if (t.size() >= prompt.size()) continue;                 // strictly shorter only
        if (best != entries_.end() && t.size() <= best->tokens.size()) continue;
        if (std::equal(t.begin(), t.end(), prompt.begin())) best = it;
    }
    PrefixHit h;
    if (best == entries_.end()) { ++misses; return h; }
    h.entry = best->id; h.tokens = (uint32_t)best->tokens.size();
    entries_.splice(entries_.begin(), entries_, best);           // most recently used
    ++hits;
    return h;
}

int64_t PrefixIndex::insert(const std::vector<int32_t>& tokens, std::vector<int64_t>& evicted) {
    if (tokens.size() < min_tokens_ || tokens.size() > capacity_ || max_entries_ == 0) { ++skipped; return -1; }
    for (auto it = entries_.begin(); it != entries_.end(); ++it)
        if (it->tokens == tokens) { entries_.splice(entries_.begin(), entries_, it); ++skipped; return -1; }
    while (!entries_.empty() && (entries_.size() >= max_entries_ || used_ + tokens.size() > capacity_)) {
        evicted.push_back(entries_.back().id);
        used_ -= (uint32_t)entries_.back().tokens.size();
        entries_.pop_back();
        ++evictions;
    }
    entries_.push_front({next_id_++, tokens});
    used_ += (uint32_t)tokens.size();
    ++inserts;
    return entries_.front().id;
}

void PrefixIndex::erase(int64_t entry) {
    for (auto it = entries_.begin(); it != entries_.end(); ++it)
        if (it->id == entry) { used_ -= (uint32_t)it->tokens.size(); entries_.erase(it); return; }
}

// ------------------------------------------------------------------------------------------------ speculative
AcceptResult spec_greedy_accept(const std::vector<int32_t>& drafts, const std::vector<int32_t>& target) {
    if (target.size() != drafts.size() + 1) throw Error(StatusCode::invalid_argument, "target must have one row more than drafts");
    uint32_t a = 0;
    while (a < drafts.size() && drafts[a] == target[a] && target[a] >= 0) ++a;
    return {a, target[a], a == drafts.size()};
}

void SpecTransaction::begin(uint32_t position, uint32_t n_rows) {
    if (state != Idle) throw Error(StatusCode::invalid_argument, "speculative round already open");
    base_position = position; rows = n_rows; accepted = 0; state = Proposed;
}
void SpecTransaction::verified(uint32_t n_accepted) {
    if (state != Proposed || n_accepted + 1 > rows) throw Error(StatusCode::invalid_argument, "bad verify transition");
    accepted = n_accepted; state = Verified;
}
uint32_t SpecTransaction::commit() {
    if (state != Verified) throw Error(StatusCode::invalid_argument, "commit before verify");
    state = Committed;
    return base_position + accepted + 1;
}
void SpecTransaction::rollback() {
    if (state != Proposed && state != Verified) throw Error(StatusCode::invalid_argument, "nothing to roll back");
    state = RolledBack;
}
void SpecTransaction::reset() { state = Idle; rows = accepted = 0; }

std::vector<int32_t> ngram_tail(const std::vector<int32_t>& h, uint32_t n, uint32_t max_tokens) {
    std::vector<int32_t> out;
    if (n == 0 || max_tokens == 0 || h.size() < (size_t)n + 1) return out;
    const size_t tail = h.size() - n;
    for (size_t start = tail; start-- > 0;) {          // latest earlier occurrence first
        if (std::equal(h.begin() + start, h.begin() + start + n, h.begin() + tail)) {
            for (size_t i = start + n; i < h.size() && out.size() < max_tokens; ++i) out.push_back(h[i]);
            break;
        }
    }
    return out;
}

uint32_t crc32(const uint8_t* data, size_t n, uint32_t seed) {
    static uint32_t table[256];
    static bool init = false;
    if (!init) {
        for (uint32_t i = 0; i < 256; ++i) {
            uint32_t c = i;
            for (int k = 0; k < 8; ++k) c = (c & 1) ? 0xEDB88320u ^ (c >> 1) : c >> 1;
            table[i] = c;
        }
        init = true;
    }
    uint32_t c = ~seed;
    for (size_t i = 0; i < n; ++i) c = table[(c ^ data[i]) & 0xFF] ^ (c >> 8);
    return ~c;
}

}  // namespace psrt

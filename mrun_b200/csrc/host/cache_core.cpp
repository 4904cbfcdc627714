// The bookkeeping of the cache manager on the host, behind a plain C interface: pools of pages
// with a free list, the block table of every state slot per group of layers, and appending as
// plan -> commit / rollback.  No device code and no tensors: the Python side owns those and hands
// the table changes queued here to the device in one scatter per step.
//
// The reference keeps the same books in its ledger (plan, do, commit:
// crates/mrun-engine/src/ledger.rs:5-9) and per-lane state (crates/mrun-engine/src/state.rs:87-151).
//
// Order matters and is part of the interface, because the tests rely on it to show that a page
// one request gave back is soon written by another: pages freed go on top of the free list in
// the order given, and are handed out from the top.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <utility>
#include <vector>

#define HOST_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr int FREED = -1;

struct Pool {
    int size = 0;
    std::vector<int> free_list;          // the top is the back
    std::vector<char> held;
    std::string error;

    explicit Pool(int n) : size(n), held(n, 0) {
        free_list.reserve(n);
        for (int p = n - 1; p >= 0; --p) free_list.push_back(p);
    }
    int free_count() const { return (int)free_list.size(); }
    // All n pages or nothing: false when fewer are free.
    bool alloc(int n, std::vector<int>& out) {
        if (n > free_count()) return false;
        for (int i = 0; i < n; ++i) {
            const int page = free_list.back();
            free_list.pop_back();
            held[page] = 1;
            out.push_back(page);
        }
        return true;
    }
    // 0 fine, 1 a page outside the pool, 2 a page freed twice; nothing changes on an error.
    int release(const int* pages, int n, int* bad) {
        for (int i = 0; i < n; ++i) {
            const int page = pages[i];
            if (page < 0 || page >= size) { *bad = page; return 1; }
            if (!held[page]) { *bad = page; return 2; }
            for (int j = 0; j < i; ++j)
                if (pages[j] == page) { *bad = page; return 2; }
        }
        for (int i = 0; i < n; ++i) {
            held[pages[i]] = 0;
            free_list.push_back(pages[i]);
        }
        return 0;
    }
    // Empty when no page is lost, listed twice, or both free and held.
    std::string check() const {
        std::vector<char> seen(size, 0);
        int held_count = 0;
        for (int page : free_list) {
            if (page < 0 || page >= size) return "a page outside the pool is on the free list";
            if (seen[page]) return "a page is on the free list twice";
            seen[page] = 1;
            if (held[page]) return "page " + std::to_string(page) + " is free and held";
        }
        for (char h : held) held_count += h ? 1 : 0;
        if (free_count() + held_count != size)
            return std::to_string(size - free_count() - held_count) + " pages lost";
        return "";
    }
};

struct Group {
    int window;                          // keys a token sees, or -1: all of them
    Pool pool;
    std::vector<int> table;              // [max_requests][max_blocks], FREED where no page is held
    std::vector<std::pair<int, int>> updates;   // (flat index, page), oldest first
    Group(int window_, int pages, int cells) : window(window_), pool(pages), table(cells, FREED) {}
};

struct Slot {
    bool live = false;
    int length = 0, pending = 0;
    std::vector<int> blocks;             // logical blocks per group
};

struct Taken {
    int slot, group, first, count;
};
struct Plan {
    std::vector<std::pair<int, int>> items;      // (slot, tokens)
    std::vector<Taken> taken;
    bool done = false;
};

struct Core {
    int page_size, num_pages, max_requests, max_blocks;
    std::vector<Group> groups;
    Pool slots;
    std::vector<Slot> state;
    std::map<int, Plan> plans;
    int next_plan = 1;
    std::string error;
    // what the last refusal for lack of room was about: group (-1: state slots, -2: blocks of a request), wanted, free
    int short_group = 0, short_wanted = 0, short_free = 0, short_slot = -1;

    Core(int n_groups, const int* windows, int page_size_, int num_pages_, int max_requests_, int max_blocks_)
        : page_size(page_size_), num_pages(num_pages_), max_requests(max_requests_), max_blocks(max_blocks_),
          slots(max_requests_), state(max_requests_) {
        groups.reserve(n_groups);
        for (int g = 0; g < n_groups; ++g) groups.emplace_back(windows[g], num_pages, max_requests * max_blocks);
        for (Slot& s : state) s.blocks.assign(n_groups, 0);
    }
    int blocks_for(int tokens) const { return (tokens + page_size - 1) / page_size; }
    void set(Group& group, int slot, int block, int page) {
        const int at = slot * max_blocks + block;
        group.table[at] = page;
        group.updates.emplace_back(at, page);
    }
    int fail(const char* format, ...) {
        char buffer[256];
        va_list args;
        va_start(args, format);
        vsnprintf(buffer, sizeof buffer, format, args);
        va_end(args);
        error = buffer;
        return -1;
    }
};

}  // namespace

// ----------------------------------------------------------------------------------------- pool
HOST_API void* mrun_pool_create(int num_pages) { return num_pages < 0 ? nullptr : new Pool(num_pages); }
HOST_API void mrun_pool_destroy(void* pool) { delete (Pool*)pool; }
HOST_API int mrun_pool_free_count(void* pool) { return ((Pool*)pool)->free_count(); }
// Writes n pages to out and returns 0, or returns 1 with nothing taken.
HOST_API int mrun_pool_alloc(void* pool, int n, int* out) {
    std::vector<int> pages;
    if (!((Pool*)pool)->alloc(n, pages)) return 1;
    if (n) std::memcpy(out, pages.data(), sizeof(int) * n);
    return 0;
}
HOST_API int mrun_pool_free(void* pool, const int* pages, int n, int* bad) { return ((Pool*)pool)->release(pages, n, bad); }
HOST_API int mrun_pool_is_held(void* pool, int page) { return ((Pool*)pool)->held[page] ? 1 : 0; }
HOST_API const char* mrun_pool_check(void* pool) {
    Pool* p = (Pool*)pool;
    p->error = p->check();
    return p->error.c_str();
}

// ----------------------------------------------------------------------------------------- core
HOST_API void* mrun_cache_create(int n_groups, const int* windows, int page_size, int num_pages, int max_requests,
                                 int max_blocks) {
    if (n_groups < 0 || page_size < 1 || num_pages < 0 || max_requests < 1 || max_blocks < 1) return nullptr;
    return new Core(n_groups, windows, page_size, num_pages, max_requests, max_blocks);
}
HOST_API void mrun_cache_destroy(void* core) { delete (Core*)core; }
HOST_API const char* mrun_cache_error(void* core) { return ((Core*)core)->error.c_str(); }
HOST_API int* mrun_cache_table(void* core, int group) { return ((Core*)core)->groups[group].table.data(); }
HOST_API int mrun_cache_free_pages(void* core, int group) { return ((Core*)core)->groups[group].pool.free_count(); }
HOST_API int mrun_cache_free_slots(void* core) { return ((Core*)core)->slots.free_count(); }
HOST_API int mrun_cache_length(void* core, int slot) { return ((Core*)core)->state[slot].length; }
HOST_API int mrun_cache_pending(void* core, int slot) { return ((Core*)core)->state[slot].pending; }
HOST_API int mrun_cache_blocks(void* core, int slot, int group) { return ((Core*)core)->state[slot].blocks[group]; }
HOST_API int mrun_cache_is_held(void* core, int group, int page) { return ((Core*)core)->groups[group].pool.held[page] ? 1 : 0; }
// What the last refusal for lack of room was about.
HOST_API void mrun_cache_shortage(void* core, int* group, int* wanted, int* free_count, int* slot) {
    Core* c = (Core*)core;
    *group = c->short_group; *wanted = c->short_wanted; *free_count = c->short_free; *slot = c->short_slot;
}

// A state slot for a new request, or -1 when none is free.
HOST_API int mrun_cache_admit(void* core) {
    Core* c = (Core*)core;
    std::vector<int> got;
    if (!c->slots.alloc(1, got)) {
        c->short_group = -1; c->short_wanted = 1; c->short_free = 0; c->short_slot = -1;
        return -1;
    }
    Slot& s = c->state[got[0]];
    s.live = true;
    s.length = s.pending = 0;
    s.blocks.assign(c->groups.size(), 0);
    return got[0];
}

// Gives back the slot and every page it holds.  0 fine, -1 with a message.
HOST_API int mrun_cache_release(void* core, int slot) {
    Core* c = (Core*)core;
    if (slot < 0 || slot >= c->max_requests || !c->state[slot].live) return c->fail("slot %d is not live", slot);
    Slot& s = c->state[slot];
    if (s.pending) return c->fail("the request in slot %d has an uncommitted step", slot);
    for (size_t g = 0; g < c->groups.size(); ++g) {
        Group& group = c->groups[g];
        std::vector<int> pages;
        for (int b = 0; b < s.blocks[g]; ++b) {
            const int page = group.table[slot * c->max_blocks + b];
            if (page != FREED) pages.push_back(page);
        }
        int bad = 0;
        if (group.pool.release(pages.data(), (int)pages.size(), &bad)) return c->fail("page %d of slot %d is not held", bad, slot);
        for (int b = 0; b < s.blocks[g]; ++b)
            if (group.table[slot * c->max_blocks + b] != FREED) c->set(group, slot, b, FREED);
        s.blocks[g] = 0;
    }
    int bad = 0;
    c->slots.release(&slot, 1, &bad);
    s.live = false;
    s.length = 0;
    return 0;
}

// Cuts the request back to its first `length` tokens (the reference trims a sequence the same
// way, crates/mrun-engine/src/ledger.rs:400-441): the pages beyond them go back, what they held is
// void, and the next step writes from position `length` on.  A group with a window refuses a cut
// that would need keys whose pages the window has already given back.
HOST_API int mrun_cache_trim(void* core, int slot, int length) {
    Core* c = (Core*)core;
    if (slot < 0 || slot >= c->max_requests || !c->state[slot].live) return c->fail("slot %d is not live", slot);
    Slot& s = c->state[slot];
    if (s.pending) return c->fail("the request in slot %d has an uncommitted step", slot);
    if (length < 0 || length > s.length) return c->fail("slot %d holds %d tokens and cannot be cut to %d", slot, s.length, length);
    const int target = c->blocks_for(length);
    for (size_t g = 0; g < c->groups.size(); ++g) {
        Group& group = c->groups[g];
        if (group.window >= 0) {
            const int low = length - group.window + 1;
            for (int b = (low > 0 ? low : 0) / c->page_size; b < target; ++b)
                if (group.table[slot * c->max_blocks + b] == FREED)
                    return c->fail("slot %d: a window of %d keys has given back what a cut to %d tokens needs", slot,
                                   group.window, length);
        }
    }
    for (size_t g = 0; g < c->groups.size(); ++g) {
        Group& group = c->groups[g];
        std::vector<int> pages;
        for (int b = target; b < s.blocks[g]; ++b) {
            const int page = group.table[slot * c->max_blocks + b];
            if (page != FREED) pages.push_back(page);
        }
        int bad = 0;
        if (group.pool.release(pages.data(), (int)pages.size(), &bad)) return c->fail("page %d of slot %d is not held", bad, slot);
        for (int b = target; b < s.blocks[g]; ++b)
            if (group.table[slot * c->max_blocks + b] != FREED) c->set(group, slot, b, FREED);
        if (s.blocks[g] > target) s.blocks[g] = target;
    }
    s.length = length;
    return 0;
}

// Takes every page the step needs: slots[i] brings tokens[i] new tokens.  Returns a plan id > 0;
// 0 when the pages (or a request's blocks) do not suffice, with nothing changed (see
// mrun_cache_shortage); -1 for a misuse, with a message.
HOST_API int mrun_cache_plan(void* core, int n, const int* slots, const int* tokens) {
    Core* c = (Core*)core;
    const int n_groups = (int)c->groups.size();
    std::vector<int> wanted(n_groups, 0);
    for (int i = 0; i < n; ++i) {
        const int slot = slots[i];
        if (slot < 0 || slot >= c->max_requests || !c->state[slot].live) return c->fail("slot %d is not live", slot);
        for (int j = 0; j < i; ++j)
            if (slots[j] == slot) return c->fail("slot %d is in the step twice", slot);
        if (tokens[i] < 1) return c->fail("slot %d: a step brings at least one token", slot);
        const Slot& s = c->state[slot];
        if (s.pending) return c->fail("the request in slot %d has an uncommitted step", slot);
        const int target = c->blocks_for(s.length + tokens[i]);
        if (n_groups && target > c->max_blocks) {
            c->short_group = -2; c->short_wanted = target; c->short_free = c->max_blocks; c->short_slot = slot;
            return 0;
        }
        for (int g = 0; g < n_groups; ++g) wanted[g] += target > s.blocks[g] ? target - s.blocks[g] : 0;
    }
    for (int g = 0; g < n_groups; ++g)
        if (wanted[g] > c->groups[g].pool.free_count()) {
            c->short_group = g; c->short_wanted = wanted[g]; c->short_free = c->groups[g].pool.free_count(); c->short_slot = -1;
            return 0;
        }
    const int id = c->next_plan++;
    Plan& plan = c->plans[id];
    for (int i = 0; i < n; ++i) {
        const int slot = slots[i];
        Slot& s = c->state[slot];
        const int target = c->blocks_for(s.length + tokens[i]);
        for (int g = 0; g < n_groups; ++g) {
            const int count = target > s.blocks[g] ? target - s.blocks[g] : 0;
            if (!count) continue;
            std::vector<int> pages;
            c->groups[g].pool.alloc(count, pages);
            const int first = s.blocks[g];
            plan.taken.push_back({slot, g, first, count});
            for (int k = 0; k < count; ++k) c->set(c->groups[g], slot, first + k, pages[k]);
            s.blocks[g] += count;
        }
        s.pending = tokens[i];
        plan.items.emplace_back(slot, tokens[i]);
    }
    return id;
}

// The step ran: the lengths advance, and a window gives back the pages it has passed.
HOST_API int mrun_cache_commit(void* core, int plan_id) {
    Core* c = (Core*)core;
    auto found = c->plans.find(plan_id);
    if (found == c->plans.end() || found->second.done) return c->fail("the plan was already committed or rolled back");
    for (const auto& item : found->second.items) {
        Slot& s = c->state[item.first];
        s.length += item.second;
        s.pending = 0;
        for (size_t g = 0; g < c->groups.size(); ++g) {
            Group& group = c->groups[g];
            if (group.window < 0) continue;
            // the next token sits at position >= length and sees keys >= length - window + 1
            const int low = s.length - group.window + 1;
            const int first_needed = (low > 0 ? low : 0) / c->page_size;
            std::vector<int> passed, pages;
            for (int b = 0; b < first_needed && b < s.blocks[g]; ++b)
                if (group.table[item.first * c->max_blocks + b] != FREED) {
                    passed.push_back(b);
                    pages.push_back(group.table[item.first * c->max_blocks + b]);
                }
            if (passed.empty()) continue;
            int bad = 0;
            group.pool.release(pages.data(), (int)pages.size(), &bad);
            for (int b : passed) c->set(group, item.first, b, FREED);
        }
    }
    c->plans.erase(found);
    return 0;
}

// The step did not run: everything the plan took goes back.
HOST_API int mrun_cache_rollback(void* core, int plan_id) {
    Core* c = (Core*)core;
    auto found = c->plans.find(plan_id);
    if (found == c->plans.end() || found->second.done) return c->fail("the plan was already committed or rolled back");
    Plan& plan = found->second;
    for (auto it = plan.taken.rbegin(); it != plan.taken.rend(); ++it) {
        Group& group = c->groups[it->group];
        Slot& s = c->state[it->slot];
        if (s.blocks[it->group] != it->first + it->count) return c->fail("slot %d changed since the plan was made", it->slot);
        std::vector<int> pages(it->count);
        for (int k = 0; k < it->count; ++k) pages[k] = group.table[it->slot * c->max_blocks + it->first + k];
        int bad = 0;
        group.pool.release(pages.data(), it->count, &bad);
        for (int k = 0; k < it->count; ++k) c->set(group, it->slot, it->first + k, FREED);
        s.blocks[it->group] = it->first;
    }
    for (const auto& item : plan.items) c->state[item.first].pending = 0;
    c->plans.erase(found);
    return 0;
}

// The queued table changes of a group, oldest index first with only the last change of an index
// kept; the queue is emptied.  Returns their number (at most `capacity` are written).
HOST_API int mrun_cache_drain(void* core, int group_id, int* index, int* value, int capacity) {
    Group& group = ((Core*)core)->groups[group_id];
    std::map<int, int> position;                         // flat index -> place in the output
    int n = 0;
    for (const auto& update : group.updates) {
        auto found = position.find(update.first);
        if (found != position.end()) {
            if (found->second < capacity) value[found->second] = update.second;
        } else {
            position[update.first] = n;
            if (n < capacity) {
                index[n] = update.first;
                value[n] = update.second;
            }
            ++n;
        }
    }
    if (n <= capacity) group.updates.clear();
    return n;
}
HOST_API int mrun_cache_pending_updates(void* core, int group_id) {
    return (int)((Core*)core)->groups[group_id].updates.size();
}

// Lays out the per-token arrays of a step: entry s brings counts[s] tokens of the request in
// slots[s], at positions length .. length + counts[s] - 1 (its pages for them are planned).
// positions, token_slot: one value per token; seg_q_start, seg_kv_len, seg_slot: one per entry;
// maps[g]: per token its place in the pages of group g (page * page_size + offset), -1 where the
// page was given back.  Returns the number of tokens, or -1 with a message.
HOST_API int mrun_cache_layout_step(void* core, int n, const int* slots, const int* counts, int* positions,
                                    int* token_slot, int* seg_q_start, int* seg_kv_len, int* seg_slot, int** maps) {
    Core* c = (Core*)core;
    int row = 0;
    for (int s = 0; s < n; ++s) {
        const int slot = slots[s];
        if (slot < 0 || slot >= c->max_requests || !c->state[slot].live) return c->fail("slot %d is not live", slot);
        const int start = c->state[slot].length, count = counts[s];
        seg_q_start[s] = row;
        seg_kv_len[s] = start + count;
        seg_slot[s] = slot;
        for (int i = 0; i < count; ++i) {
            positions[row + i] = start + i;
            token_slot[row + i] = slot;
        }
        for (size_t g = 0; g < c->groups.size(); ++g) {
            const int* pages = c->groups[g].table.data() + (size_t)slot * c->max_blocks;
            if ((start + count + c->page_size - 1) / c->page_size > c->state[slot].blocks[g])
                return c->fail("slot %d holds no pages for positions up to %d", slot, start + count - 1);
            int* map = maps[g] + row;
            for (int i = 0; i < count; ++i) {
                const int p = start + i, page = pages[p / c->page_size];
                map[i] = page == FREED ? -1 : page * c->page_size + p % c->page_size;
            }
        }
        row += count;
    }
    return row;
}

// No page lost, held by two requests, or free while held; the tables agree with the slots.
// Empty when all is well.
HOST_API const char* mrun_cache_check(void* core) {
    Core* c = (Core*)core;
    c->error = c->slots.check();
    if (!c->error.empty()) { c->error = "state slots: " + c->error; return c->error.c_str(); }
    int live = 0;
    for (const Slot& s : c->state) live += s.live ? 1 : 0;
    if (c->slots.free_count() + live != c->max_requests) { c->error = "a state slot is lost"; return c->error.c_str(); }
    for (size_t g = 0; g < c->groups.size(); ++g) {
        const Group& group = c->groups[g];
        const std::string name = "group " + std::to_string(g) + ": ";
        c->error = group.pool.check();
        if (!c->error.empty()) { c->error = name + c->error; return c->error.c_str(); }
        std::vector<char> seen(c->num_pages, 0);
        int held = 0;
        for (int slot = 0; slot < c->max_requests; ++slot) {
            const Slot& s = c->state[slot];
            const int blocks = s.live ? s.blocks[g] : 0;
            for (int b = 0; b < c->max_blocks; ++b) {
                const int page = group.table[slot * c->max_blocks + b];
                if (b >= blocks) {
                    if (page != FREED) { c->error = name + "the block table of slot " + std::to_string(slot) + " holds a page beyond the request's blocks"; return c->error.c_str(); }
                    continue;
                }
                if (page == FREED) continue;
                if (page < 0 || page >= c->num_pages || seen[page]) { c->error = name + "a page is held twice"; return c->error.c_str(); }
                seen[page] = 1;
                ++held;
                if (!group.pool.held[page]) { c->error = name + "page " + std::to_string(page) + " is in a block table and free"; return c->error.c_str(); }
            }
        }
        if (held + group.pool.free_count() != c->num_pages) {
            c->error = name + std::to_string(c->num_pages - held - group.pool.free_count()) + " pages lost";
            return c->error.c_str();
        }
    }
    c->error.clear();
    return c->error.c_str();
}

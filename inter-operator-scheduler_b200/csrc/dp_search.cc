// The dynamic-programming schedule search of IOS in native code.
//
// Counterpart of ending_iterator, dop, latency and get_stage_list of the reference
// (python/ios/optimizer.py:450-510, 513-593, 297-340, 596-606): a state is the set of operators of a
// block part that are still unscheduled, a transition removes an ENDING -- a successor-closed set that
// becomes the last stage -- which is either a set of mergeable convolutions among the sinks (one merged
// convolution) or up to max_num_groups disjoint groups, each the successor closure of one operator picked
// from the tail of a chain of a chain decomposition.  cost(s) = min over endings (cost(s - e) + latency(e)).
//
// Which endings a state has does not depend on any latency, so the search runs in two passes over the
// same depth-first traversal: the first records every candidate stage in the order in which the
// reference would first ask for its latency, the caller measures them (all at once, on several GPUs if
// it likes, structurally equal ones only once), the second evaluates the recurrence.  Enumeration order,
// memoisation by operator set and strict '<' tie-breaking follow the reference, so the same sequence of
// measurements yields the same schedule.  Operators are indexed inside their part (at most 128).
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/ios_runtime.h"

namespace ios {
void record_error(const char *message);
}

namespace {

using u128 = unsigned __int128;

struct MaskHash {
    size_t operator()(u128 v) const {
        const uint64_t lo = uint64_t(v), hi = uint64_t(v >> 64);
        uint64_t x = lo * 0x9E3779B97F4A7C15ull ^ (hi + 0xD6E8FEB86659FD93ull) * 0xC2B2AE3D27D4EB4Full;
        x ^= x >> 32;
        return size_t(x);
    }
};

inline u128 bit(int i) { return u128(1) << i; }
inline bool has(u128 m, int i) { return (m >> i) & 1; }
inline int popcount(u128 m) { return __builtin_popcountll(uint64_t(m)) + __builtin_popcountll(uint64_t(m >> 64)); }

struct Stage {
    int kind;                               // 0 merge, 1 parallel
    u128 mask;
    std::vector<std::vector<int>> groups;   // as the reference hands them to the cost model
    double latency = -1.0;
};

}  // namespace

struct ios_dp {
    int n = 0;
    std::vector<u128> succ;                 // direct successors inside the part
    std::vector<int> merge_key;             // < 0: not a convolution; else (merge class << 1) | plain
    std::vector<std::vector<int>> chains;
    bool use_merge = false, use_parallel = false;
    int max_group_size = 3, max_num_groups = 8;

    std::vector<Stage> stages;              // in order of first request
    std::unordered_map<u128, int, MaskHash> merge_index, parallel_index;
    std::unordered_map<u128, double, MaskHash> dp;
    std::unordered_map<u128, int, MaskHash> ep;       // best ending (stage index) of a state
    std::unordered_map<u128, char, MaskHash> seen;    // states visited by the enumeration pass
    long long transitions = 0;
    bool enumerated = false;
    std::vector<int> chosen;

    // successor closure (itself included) of every member of state s, inside s
    void closures(u128 s, std::vector<u128> &closure) const {
        closure.assign(size_t(n), 0);
        for (int u = n - 1; u >= 0; --u) {
            if (!has(s, u)) continue;
            u128 c = bit(u);
            u128 next = succ[u] & s;
            for (int v = u + 1; v < n && next; ++v)
                if (has(next, v)) {
                    c |= closure[v];
                    next &= ~bit(v);
                }
            closure[u] = c;
        }
    }

    int stage_of(int kind, u128 mask, const std::vector<std::vector<int>> &groups) {
        auto &index = kind == 0 ? merge_index : parallel_index;
        auto it = index.find(mask);
        if (it != index.end()) return it->second;
        Stage st;
        st.kind = kind;
        st.mask = mask;
        st.groups = groups;
        stages.push_back(st);
        index.emplace(mask, int(stages.size()) - 1);
        return int(stages.size()) - 1;
    }

    // Both passes: enumerate == true records stages (no costs yet), false evaluates the recurrence.
    double visit(u128 s, bool enumerate) {
        if (s == 0) return 0.0;
        if (enumerate) {
            if (seen.count(s)) return 0.0;
            seen.emplace(s, 1);
        } else {
            auto it = dp.find(s);
            if (it != dp.end()) return it->second;
        }
        std::vector<u128> closure;
        closures(s, closure);
        double best = 1e19;
        int best_stage = -1;
        auto consider = [&](int kind, u128 used, const std::vector<std::vector<int>> &groups) {
            const double rest = visit(s & ~used, enumerate);
            const int index = stage_of(kind, used, groups);     // (the reference asks for the latency after the recursion)
            ++transitions;
            if (enumerate) return;
            const double total = rest + stages[size_t(index)].latency;
            if (total < best) {
                best = total;
                best_stage = index;
            }
        };
        if (use_merge) {
            u128 sinks = 0;
            for (int u = 0; u < n; ++u)
                if (has(s, u) && closure[u] == bit(u)) sinks |= bit(u);
            // non-empty sub-masks in decreasing numeric order
            for (u128 sub = sinks; sub; sub = (sub - 1) & sinks) {
                bool ok = true;
                if (popcount(sub) > 1) {
                    // key >> 1 names the class (same input value, resolution, stride, activation), bit 0 says that the
                    // operator is a plain convolution of one input value; the reference compares every operator with
                    // the first of the set and asks only the others to be plain (optimizer.py:245-278)
                    int cls = -2;
                    for (int u = 0; u < n && ok; ++u)
                        if (has(sub, u)) {
                            if (merge_key[u] < 0) ok = false;
                            else if (cls == -2) cls = merge_key[u] >> 1;
                            else if (cls != (merge_key[u] >> 1) || !(merge_key[u] & 1)) ok = false;
                        }
                }
                if (!ok) continue;
                std::vector<std::vector<int>> groups;
                for (int u = 0; u < n; ++u)
                    if (has(sub, u)) groups.push_back({u});
                consider(0, sub, groups);
            }
        }
        if (use_parallel) {
            // per chain: nothing, or one of the last max_group_size operators of the chain's prefix inside s
            const size_t nc = chains.size();
            std::vector<int> begins(nc), lengths(nc);
            for (size_t i = 0; i < nc; ++i) {
                int end = 0;
                for (size_t pos = 0; pos < chains[i].size(); ++pos) {
                    if (!has(s, chains[i][pos])) break;
                    end = int(pos) + 1;
                }
                begins[i] = end - max_group_size > 0 ? end - max_group_size : 0;
                lengths[i] = end - begins[i];
            }
            std::vector<int> digit(nc, 0);
            std::vector<int> picks;
            std::vector<std::vector<int>> groups;
            bool more = nc > 0;
            while (more) {
                picks.clear();
                for (size_t i = 0; i < nc; ++i)
                    if (digit[i] != lengths[i]) picks.push_back(chains[i][size_t(begins[i] + digit[i])]);
                bool ok = !picks.empty() && int(picks.size()) <= max_num_groups;
                u128 all = 0;
                for (size_t a = 0; a < picks.size() && ok; ++a) {
                    if (all & closure[size_t(picks[a])]) ok = false;
                    all |= closure[size_t(picks[a])];
                }
                for (size_t a = 0; a < picks.size() && ok; ++a)
                    if (popcount(closure[size_t(picks[a])]) > max_group_size) ok = false;
                if (ok) {
                    groups.clear();
                    for (int u : picks) {
                        std::vector<int> group;
                        for (int v = 0; v < n; ++v)
                            if (has(closure[size_t(u)], v)) group.push_back(v);
                        groups.push_back(group);
                    }
                    consider(1, all, groups);
                }
                // next code of the mixed-radix counter, lowest digit = first chain
                size_t i = 0;
                for (; i < nc; ++i) {
                    if (++digit[i] <= lengths[i]) break;
                    digit[i] = 0;
                }
                more = i < nc;
            }
        }
        if (!enumerate) {
            dp.emplace(s, best);
            ep.emplace(s, best_stage);
        }
        return best;
    }
};

namespace {

thread_local std::string g_dp_error;

template <class F>
int guarded(F &&body) {
    try {
        body();
        ios::record_error("");
        return IOS_OK;
    } catch (const std::invalid_argument &e) {
        ios::record_error(e.what());
        return IOS_ERR_ARGUMENT;
    } catch (const std::length_error &e) {
        ios::record_error(e.what());
        return IOS_ERR_LIMIT;
    } catch (const std::exception &e) {
        ios::record_error(e.what());
        return IOS_ERR_GRAPH;
    }
}

}  // namespace

extern "C" {

int ios_dp_create(int n, const unsigned long long *succ_lo, const unsigned long long *succ_hi, const int *merge_key,
                  int num_chains, const int *chain_offsets, const int *chain_nodes, int use_merge, int use_parallel,
                  int max_group_size, int max_num_groups, ios_dp **out) {
    return guarded([&]() {
        if (!out) throw std::invalid_argument("out must not be NULL");
        *out = nullptr;
        if (n <= 0 || !succ_lo || !succ_hi || !merge_key || num_chains < 0 || (num_chains > 0 && (!chain_offsets || !chain_nodes)))
            throw std::invalid_argument("bad arguments");
        if (n > 128) throw std::length_error("limit: a part holds at most 128 operators in the native search");
        if (!use_merge && !use_parallel) throw std::invalid_argument("the search needs merge and/or parallel stages");
        if (max_group_size <= 0 || max_num_groups <= 0) throw std::invalid_argument("max_group_size and max_num_groups must be positive");
        ios_dp *h = new ios_dp;
        h->n = n;
        h->succ.resize(size_t(n));
        h->merge_key.assign(merge_key, merge_key + n);
        for (int u = 0; u < n; ++u) {
            h->succ[size_t(u)] = (u128(succ_hi[u]) << 64) | u128(succ_lo[u]);
            // operators are in topological order: successors have larger indices
            const u128 below = (bit(u) - 1) | bit(u);
            if (h->succ[size_t(u)] & below) {
                delete h;
                throw std::invalid_argument("operators must be indexed in topological order");
            }
        }
        for (int c = 0; c < num_chains; ++c) {
            std::vector<int> chain(chain_nodes + chain_offsets[c], chain_nodes + chain_offsets[c + 1]);
            for (int v : chain)
                if (v < 0 || v >= n) {
                    delete h;
                    throw std::invalid_argument("a chain names an operator outside the part");
                }
            h->chains.push_back(chain);
        }
        h->use_merge = use_merge != 0;
        h->use_parallel = use_parallel != 0;
        h->max_group_size = max_group_size;
        h->max_num_groups = max_num_groups;
        *out = h;
    });
}

int ios_dp_enumerate(ios_dp *h, int *num_stages) {
    return guarded([&]() {
        if (!h || !num_stages) throw std::invalid_argument("handle and num_stages must not be NULL");
        if (!h->enumerated) {
            const u128 full = h->n == 128 ? ~u128(0) : bit(h->n) - 1;
            h->transitions = 0;
            h->visit(full, true);
            h->enumerated = true;
        }
        *num_stages = int(h->stages.size());
    });
}

int ios_dp_stage(ios_dp *h, int index, int *kind, int *num_groups, int *group_offsets, int *nodes) {
    return guarded([&]() {
        if (!h || !kind || !num_groups || !group_offsets || !nodes) throw std::invalid_argument("arguments must not be NULL");
        if (index < 0 || index >= int(h->stages.size())) throw std::invalid_argument("stage index out of range");
        const Stage &st = h->stages[size_t(index)];
        *kind = st.kind;
        *num_groups = int(st.groups.size());
        int at = 0;
        for (size_t g = 0; g < st.groups.size(); ++g) {
            group_offsets[g] = at;
            for (int v : st.groups[g]) nodes[at++] = v;
        }
        group_offsets[st.groups.size()] = at;
    });
}

int ios_dp_set_latency(ios_dp *h, int index, double latency) {
    return guarded([&]() {
        if (!h) throw std::invalid_argument("handle must not be NULL");
        if (index < 0 || index >= int(h->stages.size())) throw std::invalid_argument("stage index out of range");
        h->stages[size_t(index)].latency = latency;
    });
}

int ios_dp_solve(ios_dp *h, int *num_chosen, double *best_cost, long long *num_states, long long *num_transitions) {
    return guarded([&]() {
        if (!h || !num_chosen) throw std::invalid_argument("handle and num_chosen must not be NULL");
        if (!h->enumerated) throw std::invalid_argument("enumerate the stages and set their latencies first");
        for (const Stage &st : h->stages)
            if (st.latency < 0.0) throw std::invalid_argument("a candidate stage has no latency yet");
        h->dp.clear();
        h->ep.clear();
        h->transitions = 0;
        const u128 full = h->n == 128 ? ~u128(0) : bit(h->n) - 1;
        const double best = h->visit(full, false);
        h->chosen.clear();
        for (u128 s = full; s;) {
            const int index = h->ep.at(s);
            if (index < 0) throw std::runtime_error("a state has no ending: the part cannot be scheduled under these limits");
            h->chosen.push_back(index);
            s &= ~h->stages[size_t(index)].mask;
        }
        // first stage first
        for (size_t i = 0, j = h->chosen.size(); i + 1 < j; ++i, --j) std::swap(h->chosen[i], h->chosen[j - 1]);
        *num_chosen = int(h->chosen.size());
        if (best_cost) *best_cost = best;
        if (num_states) *num_states = (long long)h->dp.size();
        if (num_transitions) *num_transitions = h->transitions;
    });
}

int ios_dp_chosen(ios_dp *h, int *stage_indices) {
    return guarded([&]() {
        if (!h || !stage_indices) throw std::invalid_argument("arguments must not be NULL");
        for (size_t i = 0; i < h->chosen.size(); ++i) stage_indices[i] = h->chosen[i];
    });
}

int ios_dp_destroy(ios_dp *h) {
    delete h;
    return IOS_OK;
}

}  // extern "C"

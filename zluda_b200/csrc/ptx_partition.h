// Sharding of a batch of independent modules over several GPUs (host code, no CUDA).
//
// The reference has one fan-out caller, zluda_precompile, which hands module after module to a thread pool
// (zluda_precompile/src/main.rs:57-64): modules share nothing, so a batch splits by module with no exchange step.  Here
// the split is greedy and byte-balanced - modules sorted by size, largest first, each onto the part with the fewest
// bytes so far - and every part keeps its modules in their original relative order, so that a part's text copies run
// over ascending host addresses.
#pragma once
#include <stdint.h>

#include <algorithm>
#include <functional>
#include <queue>
#include <utility>
#include <vector>

struct PtxPartition {
    std::vector<std::vector<uint32_t>> members;          // per part: indices into the caller's module list, ascending
    std::vector<std::pair<uint32_t, uint32_t>> where;    // per module: (part, position inside the part)
    std::vector<uint64_t> bytes;                         // per part
};

inline PtxPartition ptx_partition_greedy(const uint64_t* lens, uint32_t n, uint32_t n_parts) {
    PtxPartition p;
    if (n_parts == 0) n_parts = 1;
    p.members.resize(n_parts);
    p.where.resize(n);
    p.bytes.assign(n_parts, 0);
    std::vector<uint32_t> order(n);
    for (uint32_t i = 0; i < n; i++) order[i] = i;
    std::stable_sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) { return lens[a] > lens[b]; });
    typedef std::pair<uint64_t, uint32_t> Load;           // (bytes, part): the lightest part first, ties to the lower index
    std::priority_queue<Load, std::vector<Load>, std::greater<Load>> heap;
    for (uint32_t k = 0; k < n_parts; k++) heap.push(Load(0, k));
    for (uint32_t i : order) {
        Load l = heap.top();
        heap.pop();
        p.members[l.second].push_back(i);
        p.bytes[l.second] = l.first + lens[i];
        heap.push(Load(l.first + lens[i], l.second));
    }
    for (uint32_t k = 0; k < n_parts; k++) {
        std::sort(p.members[k].begin(), p.members[k].end());
        for (uint32_t j = 0; j < p.members[k].size(); j++) p.where[p.members[k][j]] = std::make_pair(k, j);
    }
    return p;
}

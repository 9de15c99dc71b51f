// Request partitioning for data-parallel decode: independent requests are spread over the GPUs
// of one box, each rank running its own replica of the engine on its shard. gpt.rs has no
// counterpart (its model path is single-sequence, crates/gpt-rs/src/inference/mod.rs:14-21); the
// unit of independence is one request, so ranks never exchange activations.
#include <algorithm>
#include <numeric>
#include <vector>

#include "common.cuh"

extern "C" {

// Longest-processing-time-first assignment. The cost of a request is the KV traffic it causes over
// the run: every decode step reads its whole context, so cost = sum_{t<steps} (prompt + t)
// = steps * prompt + steps * (steps - 1) / 2. Ties are broken by request index, then by rank, so
// every rank computes the same assignment without communication.
int gptrs_cuda_partition_requests(const int64_t* prompt_lens, int64_t n_requests, int64_t decode_steps, int n_ranks,
                                  int32_t* assignment, int64_t* rank_cost) {
    GPTRS_REQUIRE(n_requests >= 0 && n_ranks > 0 && decode_steps >= 0, "bad arguments");
    GPTRS_REQUIRE(n_requests == 0 || (prompt_lens && assignment), "null pointer");
    std::vector<int64_t> cost(n_requests), load(n_ranks, 0);
    for (int64_t i = 0; i < n_requests; ++i) {
        GPTRS_REQUIRE(prompt_lens[i] >= 0, "negative prompt length");
        cost[i] = decode_steps * prompt_lens[i] + decode_steps * (decode_steps - 1) / 2 + prompt_lens[i];
    }
    std::vector<int64_t> order(n_requests);
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) { return cost[a] > cost[b]; });
    for (int64_t i : order) {
        int best = 0;
        for (int r = 1; r < n_ranks; ++r)
            if (load[r] < load[best]) best = r;
        assignment[i] = best;
        load[best] += cost[i];
    }
    if (rank_cost)
        for (int r = 0; r < n_ranks; ++r) rank_cost[r] = load[r];
    return GPTRS_OK;
}

}  // extern "C"

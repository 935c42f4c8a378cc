// Host-side planning of a batched decode launch: how many positions a split should cover.
//
// b200kv_decode_attn_batched runs one CTA per (split, kv head, session); a session gets one split per
// ceil(max_length / num_splits) positions (rounded up to 128) and spreads its 128-position tiles evenly over them.
// A host that knows the sessions' lengths therefore chooses the positions per split, in steps of 128, through that
// pair, and the choice moves the launch time by up to 25 %: what matters is how the CTAs pack the device's CTA slots
// (two per SM).  This file holds the cost model that picks the pair; it launches nothing and needs no GPU.
// No counterpart in the reference, which keeps one session resident (tools/miinfer_cli.cpp:5663-5676).
#include "b200kv.h"

#include <algorithm>
#include <cstdint>
#include <functional>
#include <queue>
#include <vector>

namespace {

constexpr uint32_t kTile = 128;            // positions per tile of the streaming decode kernels
constexpr uint32_t kFixedTiles = 6;        // a CTA's prologue, pipeline fill, merge of its warps and tagged partial, in tile times
constexpr uint32_t kSplitSlotBudget = 1024;   // split slots of a launch (sessions x splits), as in the decode launcher
constexpr uint32_t kMaxSplits = 128;

// Makespan of the launch as the hardware dispatches it: CTAs in block order (split fastest, then kv head, then
// session), each onto the slot that frees up first.
uint64_t makespan(const std::vector<uint32_t>& durations, uint32_t slots) {
    std::priority_queue<uint64_t, std::vector<uint64_t>, std::greater<uint64_t>> free_at;
    for (uint32_t i = 0; i < slots; ++i) free_at.push(0);
    uint64_t last = 0;
    for (uint32_t d : durations) {
        const uint64_t t = free_at.top() + d;
        free_at.pop();
        free_at.push(t);
        last = std::max(last, t);
    }
    return last;
}

}  // namespace

extern "C" int b200kv_plan_batched_decode(const uint32_t* lengths, uint32_t sessions, uint32_t kv_heads, uint32_t cta_slots,
                                          uint32_t* num_splits, uint32_t* max_length) {
    if (num_splits == nullptr || max_length == nullptr || (lengths == nullptr && sessions != 0) || kv_heads == 0)
        return B200KV_ERR_INVALID;
    if (cta_slots == 0) cta_slots = 296;    // 148 SMs x 2 resident CTAs of the streaming decode kernels
    std::vector<uint32_t> live;
    live.reserve(sessions);
    for (uint32_t i = 0; i < sessions; ++i)
        if (lengths[i] > 0) live.push_back(lengths[i]);
    *num_splits = 1;
    *max_length = 0;
    if (live.empty()) return B200KV_OK;
    const uint32_t longest = *std::max_element(live.begin(), live.end());
    *max_length = longest;
    const uint32_t budget = std::max<uint32_t>(1, std::min<uint32_t>(kMaxSplits, kSplitSlotBudget / static_cast<uint32_t>(live.size())));
    const uint64_t top = (static_cast<uint64_t>(longest) + kTile - 1) / kTile * kTile;
    const uint64_t step = kTile * std::max<uint64_t>(1, (top + kTile * 64 - 1) / (kTile * 64));   // about 64 candidates at most
    bool have = false;
    uint64_t best_cost = 0;
    std::vector<uint32_t> durations;
    for (uint64_t per = std::max<uint64_t>(256, step); per < top + step; per += step) {
        const uint64_t splits = (longest + per - 1) / per;
        if (splits > budget || splits * per > 0xffffffffull) continue;
        durations.clear();
        for (uint32_t n : live) {
            const uint64_t tiles = (static_cast<uint64_t>(n) + kTile - 1) / kTile, k = (n + per - 1) / per;
            for (uint32_t h = 0; h < kv_heads; ++h)
                for (uint64_t c = 0; c < k; ++c)
                    durations.push_back(static_cast<uint32_t>(tiles * (c + 1) / k - tiles * c / k) + kFixedTiles);
        }
        // Averaged over the slot count, 8 fewer and 16 fewer: launches that filled every slot exactly measured 8 % slower
        // than launches that left a few free, and a packing that only works out at one exact count does not survive the
        // spread of real CTA times.
        uint64_t cost = 0;
        for (uint32_t less = 0; less <= 16; less += 8) cost += makespan(durations, cta_slots > less ? cta_slots - less : 1);
        if (!have || cost <= best_cost) {   // equal costs go to the larger split: fewer partials to merge
            have = true;
            best_cost = cost;
            *num_splits = static_cast<uint32_t>(splits);
            *max_length = static_cast<uint32_t>(splits * per);
        }
    }
    return B200KV_OK;
}

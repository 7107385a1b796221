// bonsai_sampler.h - the host-side token sampler of the `run` command: the arithmetic of the reference's Sampler::pick
// (runtime_vk/bonsai_forward.h:2525-2600) and its environment knobs (bonsai_forward.h:2659-2664: BONSAI_TEMP, BONSAI_TOPK,
// BONSAI_TOPP, BONSAI_REP_PENALTY, BONSAI_PRESENCE, BONSAI_FREQ; BONSAI_SEED here for the generator). Same results as
// bonsai_vk_b200/sampler.py (tests/test_sampler.py compares the two on random cases through `bonsai_run sampler-check`).
// Unlike the reference, `run` picks greedily on the device unless BONSAI_TEMP is set above zero.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <functional>
#include <numeric>
#include <utility>
#include <vector>

namespace bh {

struct Sampler {
    float temp = 0.70f, top_p = 1.0f;
    int top_k = 0;
    uint64_t rng = 88172645463325252ull;
    float rep_penalty = 1.15f, presence_penalty = 0.50f, freq_penalty = 0.0f;
    int penalty_last_n = 64;               // <= 0: the whole history

    uint64_t next_rand() {                 // xorshift64*
        rng ^= rng >> 12; rng ^= rng << 25; rng ^= rng >> 27;
        return rng * 2685821657736338717ull;
    }
    double uniform01() { return double(next_rand() >> 11) * (1.0 / 9007199254740992.0); }

    // logits with the penalties of the recent generation applied (a copy; `src` when nothing applies)
    const float *penalised(const float *src, uint32_t n, const std::vector<int> &hist, std::vector<float> &work) const {
        if (hist.empty() || (rep_penalty == 1.0f && presence_penalty == 0.0f && freq_penalty == 0.0f)) return src;
        const size_t from = penalty_last_n > 0 && hist.size() > size_t(penalty_last_n) ? hist.size() - size_t(penalty_last_n) : 0;
        std::vector<int> seen;
        for (size_t k = from; k < hist.size(); ++k) if (hist[k] >= 0 && uint32_t(hist[k]) < n) seen.push_back(hist[k]);
        if (seen.empty()) return src;
        std::sort(seen.begin(), seen.end());
        work.assign(src, src + n);
        for (size_t a = 0; a < seen.size();) {
            size_t b = a;
            while (b < seen.size() && seen[b] == seen[a]) ++b;
            float v = work[size_t(seen[a])];
            if (rep_penalty != 1.0f) v = v < 0.0f ? v * rep_penalty : v / rep_penalty;
            if (presence_penalty != 0.0f) v -= presence_penalty;
            if (freq_penalty != 0.0f) v -= freq_penalty * float(b - a);
            work[size_t(seen[a])] = v;
            a = b;
        }
        return work.data();
    }

    int pick(const float *logits, uint32_t n, const std::vector<int> &hist) {
        std::vector<float> work;
        const float *lg = penalised(logits, n, hist, work);
        uint32_t best = 0;
        for (uint32_t i = 1; i < n; ++i) if (lg[i] > lg[best]) best = i;         // first maximum
        if (temp <= 0.0f) return int(best);
        const float top = lg[best];
        float floor_v = -3.4e38f;
        if (top_k > 0 && uint32_t(top_k) < n) {                                   // the k-th largest logit is the floor
            std::vector<float> part(lg, lg + n);
            std::nth_element(part.begin(), part.begin() + (top_k - 1), part.end(), std::greater<float>());
            floor_v = part[size_t(top_k - 1)];
        }
        std::vector<double> pr(n, 0.0);
        double total = 0.0;
        for (uint32_t i = 0; i < n; ++i) {
            if (lg[i] < floor_v) continue;
            pr[i] = std::exp(double((lg[i] - top) / temp));
            total += pr[i];
        }
        if (!(total > 0.0)) return int(best);
        if (top_p < 1.0f) {
            std::vector<uint32_t> order;
            for (uint32_t i = 0; i < n; ++i) if (pr[i] > 0.0) order.push_back(i);
            std::stable_sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) { return pr[a] > pr[b]; });
            double mass = 0.0;
            size_t keep = order.size();
            for (size_t j = 0; j < order.size(); ++j) { mass += pr[order[j]] / total; if (mass >= double(top_p)) { keep = j + 1; break; } }
            for (size_t j = keep; j < order.size(); ++j) { total -= pr[order[j]]; pr[order[j]] = 0.0; }
        }
        const double u = uniform01() * total;
        double run = 0.0;
        for (uint32_t i = 0; i < n; ++i) { run += pr[i]; if (run >= u) return int(i); }
        return int(best);
    }

    // the environment knobs; returns whether sampling is asked for (a temperature above zero)
    bool from_env() {
        bool on = false;
        if (const char *v = std::getenv("BONSAI_TEMP")) { temp = float(std::atof(v)); on = temp > 0.0f; }
        if (const char *v = std::getenv("BONSAI_TOPK")) top_k = std::atoi(v);
        if (const char *v = std::getenv("BONSAI_TOPP")) top_p = float(std::atof(v));
        if (const char *v = std::getenv("BONSAI_REP_PENALTY")) rep_penalty = float(std::atof(v));
        if (const char *v = std::getenv("BONSAI_PRESENCE")) presence_penalty = float(std::atof(v));
        if (const char *v = std::getenv("BONSAI_FREQ")) freq_penalty = float(std::atof(v));
        if (const char *v = std::getenv("BONSAI_SEED")) { const unsigned long long s = std::strtoull(v, nullptr, 10); if (s) rng = s; }
        return on;
    }
};

}  // namespace bh

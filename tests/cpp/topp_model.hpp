// Sequential model of the exact top-p + draw procedure of the full-vocabulary sampler kernel
// (openvino.genai_b200/csrc/sampler_exact.cu): the same passes over the row, the same bin
// classification and the same walk (fsum_exact.cuh), with loops where the kernel has threads.
// Test infrastructure: it lets the procedure be checked on the CPU against std::sort + sequential sums.
#pragma once

#include <algorithm>
#include <cstdint>
#include <vector>

#include "fsum_exact.cuh"

namespace topp_model {

constexpr int kListCap = 4096;
constexpr uint32_t kTopCount = 96;          // the first elements change binade at almost every addition: always listed
constexpr double kMargin = 1.0 / 4096;      // relative margin of the hypotheses
constexpr double kDrawMargin = 1.0 / 512;   // wider: the draw's threshold is only known approximately in the first run

struct Result {
    uint32_t n_keep;
    float total;
    uint32_t pick_key, pick_idx;
};

struct Model {
    const float* p;
    int V;
    float min_thr;
    std::vector<uint32_t> A, C, PA, PC;
    std::vector<float> R;
    std::vector<uint16_t> next;
    std::vector<uint8_t> E, flag;
    std::vector<uint64_t> list;
    fsx::Bins b;
    fsx::Level L;
    uint32_t rest_cnt = 0;
    bool have_level = false;
    long long passes = 0;
    long long steps_made = 0;   // listed bins whose elements were composed into one step
    long long resumed = 0;      // draws that started from a checkpoint of the top-p run
    // checkpoints of the top-p run's walk over the first level (fsx::Checkpoints), as the kernel keeps them
    std::vector<float> ck_s = std::vector<float>(fsx::kBins / fsx::kCkGroup, 0.0f);
    std::vector<uint32_t> ck_cnt = std::vector<uint32_t>(fsx::kBins / fsx::kCkGroup, 0xffffffffu);
    std::vector<uint16_t> ck_j = std::vector<uint16_t>(fsx::kBins / fsx::kCkGroup, 0);
    std::vector<uint16_t> ck_li = std::vector<uint16_t>(fsx::kBins / fsx::kCkGroup, 0);
    bool ck_li_stale = false;

    Model(const float* p_, int V_, float min_thr_) : p(p_), V(V_), min_thr(min_thr_) {
        A.assign(fsx::kBins, 0); C.assign(fsx::kBins, 0); PA.assign(fsx::kBins, 0); PC.assign(fsx::kBins, 0);
        R.assign(fsx::kBins, 0.f); next.assign(fsx::kBins + 1, 0); E.assign(fsx::kBins, 0); flag.assign(fsx::kBins, 0);
        b = fsx::Bins{A.data(), C.data(), R.data(), PA.data(), PC.data(), next.data(), E.data(), flag.data()};
    }

    bool candidate(int i, uint32_t* key) const {
        const float x = p[i];
        if (!(x >= min_thr)) return false;
        *key = fsx::float_bits(x);
        return *key < L.F;
    }

    // pass R: counts and approximate masses of the level's bins
    void pass_counts() {
        ++passes;
        std::fill(C.begin(), C.end(), 0u); std::fill(R.begin(), R.end(), 0.f); std::fill(A.begin(), A.end(), 0u);
        std::fill(flag.begin(), flag.end(), (uint8_t)0); std::fill(E.begin(), E.end(), (uint8_t)0);
        rest_cnt = 0;
        list.clear();
        for (int i = 0; i < V; ++i) {
            uint32_t key;
            if (!candidate(i, &key)) continue;
            const uint32_t j = fsx::bin_of(L, key);
            if (j >= (uint32_t)fsx::kBins) { ++rest_cnt; continue; }
            ++C[j]; R[j] += p[i];
        }
    }

    // Hypotheses and list marks for bins j0 .. , given the exact sum s and count cnt before bin j0.
    // thr / limit: what the walk looks for; thr2 > 0: a second threshold expected later (the draw's).
    // Returns true when the list was emptied (the walk's list position starts over).
    bool classify(int j0, float s, uint32_t cnt, float thr, uint32_t limit, double thr2) {
        bool cleared = false;
        int room = kListCap - (int)list.size();
        if ((int)C[j0] > room) {    // make room: forget the listed bins
            list.clear();
            for (int j = 0; j < fsx::kBins; ++j)
                if (flag[j] & fsx::kBinListed) flag[j] = 0;
            room = kListCap;
            cleared = true;
        }
        double cum = (double)s;
        uint32_t cc = cnt;
        long long wanted = 0;   // marks are granted in bin order while their elements fit
        for (int j = j0; j < fsx::kBins; ++j) {
            if (C[j] == 0) continue;
            const double lo = cum, hi = cum + (double)R[j];
            const uint32_t cbefore = cc;
            cum = hi; cc += C[j];
            if (lo * (1.0 - kMargin) > (double)thr || (limit && cbefore >= limit)) continue;   // beyond what the walk can reach
            if (flag[j] & fsx::kBinListed) continue;
            uint32_t Eh;
            const bool certain = fsx::hyp_exponent(lo, hi, kMargin, &Eh);
            bool want = j == j0 || !certain || cbefore < kTopCount;
            if (lo * (1.0 - kMargin) <= (double)thr && (double)thr <= hi * (1.0 + kMargin)) want = true;
            if (thr2 > 0.0 && lo * (1.0 - kDrawMargin) <= thr2 && thr2 <= hi * (1.0 + kDrawMargin)) want = true;
            if (limit && cbefore + C[j] >= limit) want = true;
            const bool same_hyp = (flag[j] & fsx::kBinValid) && E[j] == Eh;
            if (same_hyp && (flag[j] & fsx::kBinTie)) want = true;
            if (want) {
                wanted += C[j];
                if (wanted <= room) {
                    E[j] = (uint8_t)(certain ? Eh : 0u);   // the exponent under which the bin may later be taken as one step, or none
                    flag[j] = fsx::kBinCollect;
                    continue;
                }
            }
            if (!same_hyp) { E[j] = (uint8_t)Eh; flag[j] = fsx::kBinDirty; A[j] = 0; }
        }
        return cleared;
    }

    // pass X: amounts of the dirty bins, elements of the bins to collect
    void pass_amounts() {
        ++passes;
        for (int i = 0; i < V; ++i) {
            uint32_t key;
            if (!candidate(i, &key)) continue;
            const uint32_t j = fsx::bin_of(L, key);
            if (j >= (uint32_t)fsx::kBins) continue;
            const uint8_t f = flag[j];
            if (f & fsx::kBinCollect) list.push_back(fsx::make_entry(key, (uint32_t)i));
            else if (f & fsx::kBinDirty) {
                bool tie;
                const uint32_t amount = fsx::plain_amount(p[i], fsx::amount_scale(E[j]), &tie);
                if (tie) flag[j] |= fsx::kBinTie;
                else {
                    const uint32_t old = A[j];
                    A[j] = old + amount;
                    if (old + amount >= 0x80000000u) flag[j] |= fsx::kBinTie;   // too much for one binade anyway: never taken as a whole
                }
            }
        }
        for (int j = 0; j < fsx::kBins; ++j) {
            if (flag[j] & fsx::kBinCollect) flag[j] = fsx::kBinListed;
            else if (flag[j] & fsx::kBinDirty) flag[j] = (uint8_t)((flag[j] & ~fsx::kBinDirty) | fsx::kBinValid);
        }
        std::sort(list.begin(), list.end(), std::greater<uint64_t>());
        // listed bins with a hypothesis: the composition of their elements' steps in list order (fsx::kBinStep)
        if (list.size() > kTopCount + 64) {
            for (int j = 0; j < fsx::kBins; ++j) {
                if (!(flag[j] & fsx::kBinListed)) continue;
                flag[j] = (uint8_t)(flag[j] & ~fsx::kBinStep);
                if (E[j] < 24u || E[j] > 254u) continue;
                fsx::Step st = fsx::step_identity();
                uint32_t cnt = 0;
                for (const uint64_t e : list) {
                    const uint32_t key = fsx::entry_key(e);
                    if (key >= L.F || fsx::bin_of(L, key) != (uint32_t)j) continue;
                    st = fsx::then(st, fsx::step_of(fsx::bits_float(key), E[j]));
                    ++cnt;
                }
                if (cnt == C[j] && fsx::step_packs(st)) {
                    A[j] = fsx::pack_step(st);
                    flag[j] = (uint8_t)(flag[j] | fsx::kBinStep);
                    ++steps_made;
                }
            }
        }
    }

    // prefix sums over plain bins and the next-stop table
    void prepare() {
        uint32_t pa = 0, pc = 0;
        int prev_plain_E = -1;
        std::vector<uint8_t> stop(fsx::kBins, 0);
        for (int j = 0; j < fsx::kBins; ++j) {
            if (C[j] != 0) {
                stop[j] = fsx::bin_is_stop(b, j, prev_plain_E);
                prev_plain_E = fsx::bin_plain(b, j) ? (int)E[j] : -1;
                if (stop[j]) pa = pc = 0;
                if (fsx::bin_plain(b, j)) { pa = fsx::sat_add(pa, A[j]); pc = std::min<uint64_t>((uint64_t)pc + C[j], 0x7fffffffu); }
            }
            PA[j] = pa; PC[j] = pc;
        }
        next[fsx::kBins] = (uint16_t)fsx::kBins;
        for (int j = fsx::kBins - 1; j >= 0; --j) next[j] = stop[j] ? (uint16_t)j : next[j + 1];
    }

    uint32_t lowest_index_with_key(uint32_t key) {
        ++passes;
        for (int i = 0; i < V; ++i)
            if (fsx::float_bits(p[i]) == key) return (uint32_t)i;
        return 0;
    }

    // One run of the walk from the top of the row: until the sum exceeds thr or `limit` elements are in.
    // Returns false when the row ends first (every candidate added).
    bool run(uint32_t F_top, float thr, uint32_t limit, double thr2, fsx::Walk* out) {
        fsx::Walk w{};
        w.s = 0.0f; w.cnt = 0; w.j = 0; w.li = 0;
        if (!have_level || L.F != F_top || L.sh != fsx::kTopSh) { L = fsx::Level{F_top, fsx::kTopSh}; have_level = false; }
        const bool record = limit == 0;   // the top-p run leaves checkpoints, the draw uses them
        if (limit != 0 && have_level) {
            int best = -1;
            for (int g = 0; g < fsx::kBins / fsx::kCkGroup; ++g)
                if (ck_cnt[g] != 0xffffffffu && ck_cnt[g] < limit && ck_s[g] <= thr) best = g;
            if (best >= 0 && ck_j[best] > 0) {
                w.s = ck_s[best]; w.cnt = ck_cnt[best]; w.j = ck_j[best]; w.li = ck_li_stale ? 0 : (int)ck_li[best];
                ++resumed;
            }
        }
        const fsx::Checkpoints ck{ck_s.data(), ck_cnt.data(), ck_j.data(), ck_li.data()};
        for (;;) {
            if (!have_level) { pass_counts(); have_level = true; }
            prepare();
            fsx::walk_level(w, L, b, list.data(), (int)list.size(), thr, limit, record && L.F == F_top && L.sh == fsx::kTopSh ? &ck : nullptr);
#ifdef TOPP_TRACE
            std::printf("walk: F %08x sh %d status %d j %d C %u s %a cnt %u list %zu rest %u\n", L.F, L.sh, w.status, w.j, w.j < fsx::kBins ? C[w.j] : 0u, w.s, w.cnt, list.size(), rest_cnt);
#endif
            if (w.status == fsx::kWalkFound) { *out = w; return true; }
            if (w.status == fsx::kWalkEnd) {
                const uint64_t span = (uint64_t)fsx::kBins << L.sh;
                if (rest_cnt == 0 || span >= L.F) { *out = w; return false; }
                L = fsx::Level{(uint32_t)(L.F - span), fsx::kTopSh};
                w.j = 0; w.li = 0; have_level = false;
                continue;
            }
            const int j = w.j;
            if ((int)C[j] > kListCap) {
                if (L.sh == 0) {   // one key, too many copies to list
                    const uint32_t key = L.F - 1u - (uint32_t)j;
                    bool found, by_limit = false;
                    fsx::add_repeated(w.s, w.cnt, fsx::bits_float(key), C[j], thr, limit, &found, &by_limit);
                    if (found) {
                        w.status = fsx::kWalkFound; w.hit_key = key; w.hit_idx = lowest_index_with_key(key); w.by_limit = by_limit;
                        *out = w;
                        return true;
                    }
                    w.j = j + 1;
                    // the bin is done: make the walk pass over it
                    C[j] = 0;
                    continue;
                }
                L = fsx::Level{L.F - ((uint32_t)j << L.sh), L.sh >= fsx::kSubBits ? L.sh - fsx::kSubBits : 0};
                w.j = 0; w.li = 0; have_level = false;
                continue;
            }
            if (classify(j, w.s, w.cnt, thr, limit, thr2)) { w.li = 0; ck_li_stale = true; }
            pass_amounts();
        }
    }

    Result solve(float top_p, float u) {
        float pmax = 0.0f;
        for (int i = 0; i < V; ++i) if (p[i] >= min_thr && p[i] > pmax) pmax = p[i];
        const uint32_t F_top = fsx::float_bits(pmax) + 1u;
        fsx::Walk w1{}, w2{};
        const bool hit = run(F_top, top_p, 0, (double)u * (double)top_p, &w1);
        (void)hit;   // when the row ends first every candidate is kept
        Result r;
        r.n_keep = w1.cnt; r.total = w1.s;
        const float rr = r.total * u;
        run(F_top, rr, r.n_keep, 0.0, &w2);
        r.pick_key = w2.hit_key; r.pick_idx = w2.hit_idx;
        return r;
    }
};

}  // namespace topp_model

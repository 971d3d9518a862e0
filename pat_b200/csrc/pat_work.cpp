// Work-list builder; see pat_work.h.
#include "pat_work.h"

#include <algorithm>
#include <cstring>
#include <numeric>
#include <unordered_map>

namespace pat {

namespace {

inline uint64_t mix64(uint64_t h, uint64_t v) {
    h ^= v + 0x9e3779b97f4a7c15ULL + (h << 6) + (h >> 2);
    h *= 0xff51afd7ed558ccdULL;
    h ^= h >> 33;
    return h;
}

struct FusedBox {            // boxes that share one page list
    const int32_t* pages;
    int num_pages;
    int kv_len;
    std::vector<int32_t> queries;
};

using Segment = WorkSegment;  // pages attended by exactly the same fused boxes

inline int ceil_div(int64_t a, int64_t b) { return static_cast<int>((a + b - 1) / b); }

}  // namespace

int WorkList::build(const PlanBucketView* buckets, int num_buckets, int batch, int hratio, int kv_heads,
                    int page_size, int64_t num_cache_pages, const WorkOptions& opt) {
    header_ = WorkHeader{};
    blob_.clear();
    grow_.clear();
    if (num_buckets < 0 || batch <= 0 || hratio < 1 || hratio > 16 || kv_heads < 1 || page_size < 16 ||
        page_size % 16 != 0 || opt.stream_rows < hratio || (num_buckets > 0 && !buckets))
        return -1;

    // ---- 1. fuse boxes with identical page lists -----------------------------
    std::vector<FusedBox> fused;
    std::unordered_map<uint64_t, std::vector<int>> by_hash;
    for (int b = 0; b < num_buckets; ++b) {
        const PlanBucketView& bk = buckets[b];
        for (int c = 0; c < bk.ctas; ++c) {
            const int nq = bk.num_seqs[c];
            const int kv = bk.kv_lens[c];
            if (nq <= 0 || kv <= 0) continue;   // nothing to attend: contributes no partial
            const int np = ceil_div(kv, page_size);
            if (nq > bk.q_stride || np > bk.block_stride) return -2;
            const int32_t* q = bk.q_table + static_cast<size_t>(c) * bk.q_stride;
            const int32_t* pg = bk.block_table + static_cast<size_t>(c) * bk.block_stride;
            for (int i = 0; i < nq; ++i)
                if (q[i] < 0 || q[i] >= batch) return -3;
            uint64_t h = mix64(0x1234, static_cast<uint64_t>(kv));
            for (int i = 0; i < np; ++i) {
                if (pg[i] < 0 || (num_cache_pages > 0 && pg[i] >= num_cache_pages)) return -4;
                h = mix64(h, static_cast<uint64_t>(pg[i]));
            }
            int found = -1;
            auto& cand = by_hash[h];
            for (int g : cand) {
                const FusedBox& f = fused[g];
                if (f.num_pages == np && f.kv_len == kv && std::memcmp(f.pages, pg, sizeof(int32_t) * np) == 0) {
                    found = g;
                    break;
                }
            }
            if (found < 0) {
                found = static_cast<int>(fused.size());
                fused.push_back(FusedBox{pg, np, kv, {}});
                cand.push_back(found);
            }
            fused[found].queries.insert(fused[found].queries.end(), q, q + nq);
        }
    }

    // ---- 2. which fused boxes contain each (page, valid) ---------------------
    // Signatures are kept as linked lists in a flat pool; their hash is updated
    // as boxes are appended (boxes are visited in increasing order, so equal
    // sets give equal sequences).
    // Full pages (all but the last page of a box, at most) are looked up in a flat table indexed
    // by page id; only partial pages go through the hash map.
    std::unordered_map<uint64_t, int> slot_of;   // (page << 32 | valid) -> slot, partial pages
    std::vector<uint64_t> slot_key, slot_hash;
    std::vector<int> slot_head, slot_tail, slot_len;
    std::vector<int> link_box, link_next;
    size_t total_links = 0;
    int32_t max_page = -1;
    for (const FusedBox& f : fused) {
        total_links += static_cast<size_t>(f.num_pages);
        for (int p = 0; p < f.num_pages; ++p) max_page = std::max(max_page, f.pages[p]);
    }
    std::vector<int> full_slot(static_cast<size_t>(max_page) + 1, -1);
    slot_key.reserve(total_links);
    slot_hash.reserve(total_links);
    slot_head.reserve(total_links);
    slot_tail.reserve(total_links);
    slot_len.reserve(total_links);
    link_box.reserve(total_links);
    link_next.reserve(total_links);
    for (int g = 0; g < static_cast<int>(fused.size()); ++g) {
        const FusedBox& f = fused[g];
        for (int p = 0; p < f.num_pages; ++p) {
            const int valid = (p == f.num_pages - 1) ? f.kv_len - p * page_size : page_size;
            const uint64_t key = (static_cast<uint64_t>(static_cast<uint32_t>(f.pages[p])) << 32) |
                                 static_cast<uint32_t>(valid);
            int s;
            bool fresh;
            if (valid == page_size) {
                int& ref = full_slot[f.pages[p]];
                fresh = ref < 0;
                if (fresh) ref = static_cast<int>(slot_key.size());
                s = ref;
            } else {
                auto ins = slot_of.emplace(key, static_cast<int>(slot_key.size()));
                s = ins.first->second;
                fresh = ins.second;
            }
            if (fresh) {
                slot_key.push_back(key);
                slot_hash.push_back(0x9876);
                slot_head.push_back(-1);
                slot_tail.push_back(-1);
                slot_len.push_back(0);
            }
            const int link = static_cast<int>(link_box.size());
            link_box.push_back(g);
            link_next.push_back(-1);
            if (slot_tail[s] >= 0) link_next[slot_tail[s]] = link; else slot_head[s] = link;
            slot_tail[s] = link;
            slot_len[s] += 1;
            slot_hash[s] = mix64(slot_hash[s], static_cast<uint64_t>(g));
        }
    }

    // ---- 3. segments = slots with the same signature -------------------------
    std::vector<Segment> segs;
    std::vector<int> seg_rep;   // a representative slot per segment (for comparing signatures)
    std::unordered_map<uint64_t, std::vector<int>> seg_by_hash;
    auto same_sig = [&](int a, int b) {
        if (slot_len[a] != slot_len[b]) return false;
        int la = slot_head[a], lb = slot_head[b];
        while (la >= 0) {
            if (link_box[la] != link_box[lb]) return false;
            la = link_next[la];
            lb = link_next[lb];
        }
        return true;
    };
    int last_seg = -1;
    uint64_t last_hash = 0;
    for (int s = 0; s < static_cast<int>(slot_key.size()); ++s) {
        const int valid = static_cast<int>(slot_key[s] & 0xffffffffu);
        const int32_t page = static_cast<int32_t>(slot_key[s] >> 32);
        // a partial page always gets a segment key of its own signature hash so that
        // two partial pages never land in one segment
        uint64_t h = slot_hash[s];
        int seg = -1;
        // consecutive pages of a box nearly always share their signature: try the segment of the
        // previous slot before the hash map
        if (last_seg >= 0 && h == last_hash && same_sig(seg_rep[last_seg], s) &&
            !(valid < page_size && segs[last_seg].partial_tokens > 0))
            seg = last_seg;
        if (seg < 0) {
            for (int c : seg_by_hash[h]) {
                if (same_sig(seg_rep[c], s) && !(valid < page_size && segs[c].partial_tokens > 0)) {
                    seg = c;
                    break;
                }
            }
        }
        if (seg < 0) {
            seg = static_cast<int>(segs.size());
            segs.emplace_back();
            seg_rep.push_back(s);
            seg_by_hash[h].push_back(seg);
            for (int l = slot_head[s]; l >= 0; l = link_next[l]) {
                const auto& q = fused[link_box[l]].queries;
                segs[seg].queries.insert(segs[seg].queries.end(), q.begin(), q.end());
            }
        }
        last_seg = seg;
        last_hash = h;
        Segment& sg = segs[seg];
        if (valid < page_size) {
            sg.partial_tokens = valid;      // appended after the loop, so that it is last
            sg.pages.push_back(-1 - page);  // marker, fixed below
        } else {
            sg.pages.push_back(page);
        }
        sg.tokens += valid;
    }
    for (Segment& sg : segs) {
        if (sg.partial_tokens > 0) {
            auto it = std::find_if(sg.pages.begin(), sg.pages.end(), [](int32_t v) { return v < 0; });
            const int32_t page = -1 - *it;
            sg.pages.erase(it);
            sg.pages.push_back(page);
        }
    }

    return finish(segs, batch, hratio, kv_heads, page_size, opt);
}

int WorkList::build_from_tree(const Tree& tree, int hratio, int kv_heads, int64_t num_cache_pages,
                              const WorkOptions& opt, int q_per_req) {
    header_ = WorkHeader{};
    blob_.clear();
    grow_.clear();
    const int batch = tree.batch(), page_size = tree.block_size();
    if (batch <= 0 || hratio < 1 || hratio > 16 || kv_heads < 1 || page_size < 16 || page_size % 16 != 0 ||
        opt.stream_rows < hratio || q_per_req < 1 || q_per_req > 64)
        return -1;
    const std::vector<TreeNode>& nodes = tree.nodes();
    const int T = q_per_req;
    // tokens on the path from the root to each node's parent (nodes are created parents first,
    // except that a split inserts the new parent after its child: walk up instead of indexing)
    std::vector<int64_t> start(nodes.size(), -1);
    auto start_of = [&](int n) {
        // iterative: climb to the first node whose start is known, then fill back down
        std::vector<int> chain;
        int at = n;
        while (at > 0 && start[at] < 0) { chain.push_back(at); at = nodes[at].parent; }
        int64_t s = at > 0 ? start[at] + nodes[at].length : 0;
        // `s` is the start of the children of `at`; chain holds the path downwards in reverse
        for (auto it = chain.rbegin(); it != chain.rend(); ++it) { start[*it] = s; s += nodes[*it].length; }
        return start[n];
    };
    std::vector<Segment> segs;
    segs.reserve(nodes.size());
    for (size_t n = 1; n < nodes.size(); ++n) {
        const TreeNode& node = nodes[n];
        if (node.length <= 0 || node.seq_indices.empty() || !node.pages) continue;
        const int np = ceil_div(node.length, page_size);
        Segment sg;
        for (int32_t q : node.seq_indices)
            if (q < 0 || q >= batch) return -3;
        if (T == 1) {
            sg.queries.assign(node.seq_indices.begin(), node.seq_indices.end());
        } else {
            // one query per (request, position); position t of a request of length L sees the first
            // L - T + 1 + t tokens of the request, hence this many of the segment's
            const int64_t s0 = start_of(static_cast<int>(n));
            bool all_full = true;
            for (int32_t q : node.seq_indices) {
                for (int t = 0; t < T; ++t) {
                    const int64_t visible = static_cast<int64_t>(tree.seq_len(q)) - T + 1 + t - s0;
                    const int32_t lim = static_cast<int32_t>(std::max<int64_t>(0, std::min<int64_t>(visible, node.length)));
                    sg.queries.push_back(q * T + t);
                    sg.limits.push_back(lim);
                    all_full = all_full && lim == node.length;
                }
            }
            if (all_full) sg.limits.clear();
        }
        sg.pages.assign(node.pages, node.pages + np);
        for (int32_t pg : sg.pages)
            if (pg < 0 || (num_cache_pages > 0 && pg >= num_cache_pages)) return -4;
        sg.tokens = node.length;
        sg.partial_tokens = node.length % page_size;
        const int only = (T == 1 && sg.queries.size() == 1) ? sg.queries[0] : -1;
        if (only >= 0 && node.children.empty() && tree.leaf_of(only) == static_cast<int>(n)) sg.owner = only;
        segs.push_back(std::move(sg));
    }
    const int rc = finish(segs, batch * T, hratio, kv_heads, page_size, opt);
    header_.q_per_req = T;
    return rc;
}

int WorkList::finish(std::vector<Segment>& segs, int batch, int hratio, int kv_heads, int page_size,
                     const WorkOptions& opt) {
    // ---- 4. classes and chunk sizes ---------------------------------------------
    const int q_per_stream = std::max(1, opt.stream_rows / hratio);
    const int q_per_dense = opt.dense_rows > 0 ? std::max(1, opt.dense_rows / hratio) : 0;
    auto is_dense = [&](const Segment& sg) {
        return q_per_dense > 0 && static_cast<int64_t>(sg.queries.size()) * hratio >= opt.dense_min_rows;
    };
    int64_t stream_cost = 0, unique_tokens = 0;
    for (const Segment& sg : segs) {
        unique_tokens += sg.tokens;
        const int nq = static_cast<int>(sg.queries.size());
        if (is_dense(sg)) {
            header_.dense_unique_tokens += sg.tokens;
        } else {
            stream_cost += sg.tokens * ceil_div(nq, q_per_stream);
            header_.stream_unique_tokens += sg.tokens;
        }
    }
    int64_t want = stream_cost * kv_heads / std::max<int64_t>(1, static_cast<int64_t>(opt.num_sms) * opt.items_per_sm);
    want = (want + page_size - 1) / page_size * page_size;
    want = std::max<int64_t>(want, std::max(opt.chunk_tokens_min, page_size));
    want = std::min<int64_t>(want, std::max(opt.chunk_tokens_max, page_size));
    const int stream_chunk = static_cast<int>(want);

    std::vector<int32_t> queries_sec, pages_sec, limits_sec;
    bool any_limits = false;
    for (const Segment& sg : segs) any_limits = any_limits || !sg.limits.empty();
    for (Segment& sg : segs) {
        sg.q_off = static_cast<int32_t>(queries_sec.size());
        queries_sec.insert(queries_sec.end(), sg.queries.begin(), sg.queries.end());
        if (any_limits) {
            if (sg.limits.empty()) limits_sec.insert(limits_sec.end(), sg.queries.size(), static_cast<int32_t>(sg.tokens));
            else limits_sec.insert(limits_sec.end(), sg.limits.begin(), sg.limits.end());
        }
        sg.page_off = static_cast<int32_t>(pages_sec.size());
        pages_sec.insert(pages_sec.end(), sg.pages.begin(), sg.pages.end());
        // room to grow in place; a dense segment is never extended (its owner would need >= 17 rows)
        if (sg.owner >= 0 && !is_dense(sg)) pages_sec.insert(pages_sec.end(), std::max(0, opt.grow_slack_pages), 0);
    }

    // ---- 5. streaming items -----------------------------------------------------
    std::vector<WorkItem> stream_items, dense_items;
    int32_t num_entries = 0;
    std::vector<int32_t> per_list(static_cast<size_t>(batch) * kv_heads, 0);
    for (const Segment& sg : segs) {
        if (is_dense(sg)) continue;
        const int nq = static_cast<int>(sg.queries.size());
        const int np = static_cast<int>(sg.pages.size());
        const int kparts = std::max(1, ceil_div(sg.tokens, stream_chunk));
        const int ppc = ceil_div(np, kparts);            // pages per KV chunk
        for (int p0 = 0; p0 < np; p0 += ppc) {
            const int p1 = std::min(np, p0 + ppc);
            const int64_t tok_lo = static_cast<int64_t>(p0) * page_size;
            const int kv = static_cast<int>(std::min<int64_t>(sg.tokens - tok_lo,
                                                              static_cast<int64_t>(p1 - p0) * page_size));
            for (int q0 = 0; q0 < nq; q0 += q_per_stream) {
                WorkItem it{};
                it.q_off = sg.q_off + q0;
                it.nq = std::min(q_per_stream, nq - q0);
                it.page_off = sg.page_off + p0;
                it.kv_len = kv;
                it.entry_base = num_entries;
                // the item that holds the last tokens of a segment one request owns is remembered
                // (through the sort below, as a head number <= -2) as the item WorkList::advance extends
                it.kv_head = (sg.owner >= 0 && p1 == np) ? -(sg.owner + 2) : -1;
                it.cost = kv;
                it.tok_lo = static_cast<int32_t>(tok_lo);
                num_entries += it.nq * kv_heads;
                for (int i = 0; i < it.nq; ++i)
                    for (int h = 0; h < kv_heads; ++h)
                        per_list[static_cast<size_t>(sg.queries[q0 + i]) * kv_heads + h] += 1;
                stream_items.push_back(it);
                header_.stream_tokens += kv;
            }
        }
    }
    std::stable_sort(stream_items.begin(), stream_items.end(),
                     [](const WorkItem& a, const WorkItem& b) { return a.cost > b.cost; });
    bool any_owner = false;
    for (const Segment& sg : segs) any_owner = any_owner || sg.owner >= 0;
    if (any_owner) {
        grow_.assign(static_cast<size_t>(batch), GrowSlot{});
        for (size_t i = 0; i < stream_items.size(); ++i) {
            WorkItem& it = stream_items[i];
            if (it.kv_head <= -2) grow_[-it.kv_head - 2].item = static_cast<int32_t>(i);
        }
        for (const Segment& sg : segs) {
            if (sg.owner < 0 || is_dense(sg)) continue;
            GrowSlot& g = grow_[sg.owner];
            g.next_page = sg.page_off + static_cast<int32_t>(sg.pages.size());     // made absolute once the blob is laid out
            g.slack = std::max(0, opt.grow_slack_pages);
            g.last_tokens = sg.partial_tokens > 0 ? sg.partial_tokens : page_size;
        }
    }
    for (WorkItem& it : stream_items) it.kv_head = -1;

    // ---- 6. dense items: equal work per persistent CTA ------------------------------
    // The dense kernel runs `shares` x kv_heads x row_lanes persistent CTAs
    // (CTA id = (share * kv_heads + head) * row_lanes + lane); every KV head gets the same
    // placement of (token range, 128-row chunk) jobs on its shares x row_lanes CTAs.
    struct DenseSeg { const Segment* sg; int chunks; };
    std::vector<DenseSeg> dsegs;
    int max_chunks = 1;
    for (const Segment& sg : segs) {
        if (!is_dense(sg)) continue;
        const int chunks = ceil_div(static_cast<int64_t>(sg.queries.size()), q_per_dense);
        dsegs.push_back(DenseSeg{&sg, chunks});
        max_chunks = std::max(max_chunks, chunks);
        header_.dense_tokens += sg.tokens * chunks;
    }
    const int row_lanes = std::min(2, max_chunks);
    std::vector<int32_t> cta_begin;
    if (!dsegs.empty()) {
        // cuts fall on multiples of `granule` tokens from the start of a segment, so that every
        // piece starts on a page boundary and on a 64-token tile boundary
        int64_t granule = 64;
        while (granule % page_size != 0) granule += 64;
        const int64_t min_piece = std::max<int64_t>(granule, opt.dense_piece_tokens_min);
        // cost unit: tokens x row chunks (what the row lanes of a share work off together); every
        // item costs about as much as kItemTokens more tokens (pipeline fill, epilogue)
        constexpr int64_t kItemTokens = 384;
        auto passes = [&](const DenseSeg& d) { return static_cast<int64_t>(d.chunks); };
        int64_t total_cost = 0;
        for (const DenseSeg& d : dsegs) total_cost += (d.sg->tokens + kItemTokens) * passes(d);
        const int64_t max_shares = std::max<int64_t>(1, opt.num_sms / (static_cast<int64_t>(kv_heads) * row_lanes));
        int64_t share_limit = max_shares;
        if (opt.dense_tile_ns > 0 && header_.stream_tokens > 0) {
            // Both kernels run at the same time: the dense CTAs hold their SMs for as long as they
            // run, the streaming kernel fills the others and takes every SM over as dense CTAs
            // retire.  Every dense CTA costs a fixed time and every share adds items, so few CTAs
            // waste the least SM time - as long as the dense kernel is not what the step waits
            // for.  The dense kernel therefore gets the fewest shares with which its estimated time
            // stays below kShare of the estimated step (the streaming kernel alone plus the SM
            // time the dense CTAs take away from it).  Too few CTAs cost far more than too many,
            // and the dense kernel is slower beside the streaming kernel than alone: hence the
            // margin.  Estimates, calibrated on a B200 (kernels timed alone, 4-148 dense CTAs on
            // five workloads): dense = kFixedNs + (tiles x dense_tile_ns + items x kItemNs) / CTAs;
            // streaming = kStreamFixedNs + kStreamPsPerTokenHead per token and KV head.
            constexpr double kStreamPsPerTokenHead = 75.0, kStreamFixedNs = 12000.0, kShare = 0.6;
            constexpr double kItemNs = 4500.0, kFixedNs = 8000.0;   // per dense item (fill, hand-over, epilogue), per launch
            const double stream_ns = kStreamFixedNs + static_cast<double>(header_.stream_tokens) * kv_heads *
                                                          kStreamPsPerTokenHead * 1e-3;
            const int64_t group = static_cast<int64_t>(kv_heads) * row_lanes;      // CTAs per share
            int64_t chunk_sum = 0, token_chunks = 0;
            for (const DenseSeg& d : dsegs) {
                chunk_sum += d.chunks;
                token_chunks += d.sg->tokens * d.chunks;
            }
            const double tile_ns = static_cast<double>(token_chunks) * kv_heads / 128.0 * opt.dense_tile_ns;
            for (int64_t sh = 1; sh < max_shares; ++sh) {
                const double ctas = static_cast<double>(sh * group);
                const double items = static_cast<double>(chunk_sum * kv_heads) + ctas;     // every share adds about one item per CTA
                const double dense_ns = kFixedNs + (tile_ns + items * kItemNs) / ctas;
                if (dense_ns <= kShare * (stream_ns + dense_ns * ctas / opt.num_sms)) {
                    share_limit = sh;
                    break;
                }
            }
        }
        const int64_t shares = std::min<int64_t>(share_limit, std::max<int64_t>(1, total_cost / row_lanes / min_piece));
        // Jobs: one per (piece, 128-row chunk), placed on the CTAs (share x row lane; the same
        // placement for every KV head).
        //  * Long segments - thousands of tokens, one chunk a good part of a CTA's fair share - are
        //    cut along their tokens: they are laid end to end and one
        //    share after the other is filled up to the fair load, cutting on granule boundaries;
        //    inside a share every chunk goes to the row lane with the least work so far, so the
        //    chunks of one piece run side by side (a 2 KB cache row - all heads of a token - is then
        //    fetched from HBM within a short window and the second row chunk finds it in L2).
        //  * Short segments - the nodes of a deep tree - stay whole, since every cut costs another
        //    item: their chunks go, longest first, to the CTA with the least work so far.
        struct Job { const DenseSeg* d; int chunk; int64_t pos, take; };
        const int64_t bins = shares * row_lanes;
        const int64_t fair = (total_cost + bins - 1) / bins;
        std::vector<std::vector<Job>> bin_jobs(static_cast<size_t>(bins));
        std::vector<int64_t> load(static_cast<size_t>(bins), 0);
        std::vector<DenseSeg> long_segs, short_segs;
        for (const DenseSeg& d : dsegs) {
            const bool is_long = d.sg->tokens + kItemTokens > fair / 4 && d.sg->tokens >= 4 * kItemTokens;
            (is_long ? long_segs : short_segs).push_back(d);
        }
        if (!long_segs.empty()) {
            struct Piece { const DenseSeg* d; int64_t pos, take; };
            std::vector<std::vector<Piece>> share_pieces;
            auto cut = [&](int64_t target) {
                share_pieces.assign(1, {});
                int64_t used = 0;
                for (const DenseSeg& d : long_segs) {
                    const int64_t tokens = d.sg->tokens, w = passes(d);
                    int64_t pos = 0;
                    while (pos < tokens) {
                        int64_t cap = (target - used) / w - kItemTokens;            // tokens of this segment that still fit
                        cap = cap / granule * granule;
                        if (cap < granule && used > 0) {                            // full: open the next share
                            share_pieces.emplace_back();
                            used = 0;
                            continue;
                        }
                        int64_t take = std::min(tokens - pos, std::max(cap, granule));
                        // do not leave a sliver behind
                        if (tokens - pos - take > 0 && tokens - pos - take < granule) take = tokens - pos;
                        share_pieces.back().push_back(Piece{&d, pos, take});
                        used += (take + kItemTokens) * w;
                        pos += take;
                    }
                }
                return static_cast<int64_t>(share_pieces.size());
            };
            int64_t target = fair * row_lanes;
            while (cut(target) > shares) target += std::max<int64_t>(target / 32, 1);
            for (size_t sh = 0; sh < share_pieces.size(); ++sh) {
                for (const Piece& pc : share_pieces[sh]) {
                    for (int chunk = 0; chunk < pc.d->chunks; ++chunk) {
                        size_t best = sh * row_lanes;
                        for (size_t b = best + 1; b < (sh + 1) * row_lanes; ++b)
                            if (load[b] < load[best]) best = b;
                        bin_jobs[best].push_back(Job{pc.d, chunk, pc.pos, pc.take});
                        load[best] += pc.take + kItemTokens;
                    }
                }
            }
        }
        {
            std::vector<Job> jobs;
            for (const DenseSeg& d : short_segs)
                for (int chunk = 0; chunk < d.chunks; ++chunk) jobs.push_back(Job{&d, chunk, 0, d.sg->tokens});
            std::stable_sort(jobs.begin(), jobs.end(), [](const Job& a, const Job& b) { return a.take > b.take; });
            for (const Job& job : jobs) {
                size_t best = 0;
                for (size_t b = 1; b < load.size(); ++b)
                    if (load[b] < load[best]) best = b;
                bin_jobs[best].push_back(job);
                load[best] += job.take + kItemTokens;
            }
        }
        for (int64_t share = 0; share < shares; ++share) {
            for (int h = 0; h < kv_heads; ++h) {
                for (int lane = 0; lane < row_lanes; ++lane) {
                    cta_begin.push_back(static_cast<int32_t>(dense_items.size()));
                    for (const Job& job : bin_jobs[static_cast<size_t>(share * row_lanes + lane)]) {
                        const Segment* sg = job.d->sg;
                        const int nq_all = static_cast<int>(sg->queries.size());
                        const int q0 = job.chunk * q_per_dense;
                        WorkItem it{};
                        it.q_off = sg->q_off + q0;
                        it.nq = std::min(q_per_dense, nq_all - q0);
                        it.page_off = sg->page_off + static_cast<int32_t>(job.pos / page_size);
                        it.kv_len = static_cast<int32_t>(job.take);
                        it.entry_base = num_entries;
                        it.kv_head = h;
                        it.cost = static_cast<int32_t>(job.take);
                        it.tok_lo = static_cast<int32_t>(job.pos);
                        num_entries += it.nq;
                        for (int i = 0; i < it.nq; ++i)
                            per_list[static_cast<size_t>(sg->queries[q0 + i]) * kv_heads + h] += 1;
                        dense_items.push_back(it);
                    }
                }
            }
        }
        cta_begin.push_back(static_cast<int32_t>(dense_items.size()));
    }
    const int num_dense_ctas = cta_begin.empty() ? 0 : static_cast<int>(cta_begin.size()) - 1;

    // ---- 7. merge lists per (request, KV head) ------------------------------------
    const size_t n_lists = static_cast<size_t>(batch) * kv_heads;
    std::vector<int32_t> indptr(n_lists + 1, 0);
    for (size_t i = 0; i < n_lists; ++i) indptr[i + 1] = indptr[i] + per_list[i];
    std::vector<int32_t> fill(indptr.begin(), indptr.end() - 1);
    std::vector<int32_t> entries(indptr[n_lists], 0);
    for (const WorkItem& it : stream_items)
        for (int i = 0; i < it.nq; ++i)
            for (int h = 0; h < kv_heads; ++h)
                entries[fill[static_cast<size_t>(queries_sec[it.q_off + i]) * kv_heads + h]++] = it.entry_base + i * kv_heads + h;
    for (const WorkItem& it : dense_items)
        for (int i = 0; i < it.nq; ++i)
            entries[fill[static_cast<size_t>(queries_sec[it.q_off + i]) * kv_heads + it.kv_head]++] = it.entry_base + i;
    int max_per_list = 0;
    for (size_t i = 0; i < n_lists; ++i) {
        std::sort(entries.begin() + indptr[i], entries.begin() + indptr[i + 1]);   // deterministic merge order
        max_per_list = std::max(max_per_list, per_list[i]);
    }

    // ---- 8. blob ------------------------------------------------------------------
    const size_t n_items = stream_items.size() + dense_items.size();
    auto align8 = [](size_t v) { return (v + 7) / 8 * 8; };
    const size_t items_off = 0;
    const size_t queries_off = align8(items_off + n_items * 8);
    const size_t limits_off = align8(queries_off + queries_sec.size());
    const size_t dense_q_off = align8(limits_off + limits_sec.size());
    const size_t dense_q_width = static_cast<size_t>(std::max(1, q_per_dense));
    const size_t pages_off = align8(dense_q_off + dense_items.size() * dense_q_width);
    const size_t cta_off = align8(pages_off + pages_sec.size());
    const size_t indptr_off = align8(cta_off + cta_begin.size());
    const size_t entries_off = align8(indptr_off + indptr.size());
    const size_t total = align8(entries_off + entries.size()) + 8;
    blob_.assign(total, 0);
    if (!stream_items.empty())
        std::memcpy(blob_.data() + items_off, stream_items.data(), stream_items.size() * sizeof(WorkItem));
    if (!dense_items.empty())
        std::memcpy(blob_.data() + items_off + stream_items.size() * 8, dense_items.data(),
                    dense_items.size() * sizeof(WorkItem));
    std::copy(queries_sec.begin(), queries_sec.end(), blob_.begin() + queries_off);
    std::copy(limits_sec.begin(), limits_sec.end(), blob_.begin() + limits_off);
    for (size_t d = 0; d < dense_items.size(); ++d) {
        int32_t* row = blob_.data() + dense_q_off + d * dense_q_width;
        const WorkItem& it = dense_items[d];
        for (size_t i = 0; i < dense_q_width; ++i)
            row[i] = static_cast<int>(i) < it.nq ? queries_sec[it.q_off + i] : -1;
    }
    std::copy(pages_sec.begin(), pages_sec.end(), blob_.begin() + pages_off);
    std::copy(cta_begin.begin(), cta_begin.end(), blob_.begin() + cta_off);
    std::copy(indptr.begin(), indptr.end(), blob_.begin() + indptr_off);
    std::copy(entries.begin(), entries.end(), blob_.begin() + entries_off);

    header_.batch = batch;
    header_.hratio = hratio;
    header_.page_size = page_size;
    header_.kv_heads = kv_heads;
    header_.num_stream_items = static_cast<int32_t>(stream_items.size());
    header_.num_dense_items = static_cast<int32_t>(dense_items.size());
    header_.num_dense_ctas = num_dense_ctas;
    header_.num_entries = num_entries;
    header_.max_entries_per_list = max_per_list;
    header_.items_off = static_cast<int32_t>(items_off);
    header_.queries_off = static_cast<int32_t>(queries_off);
    header_.pages_off = static_cast<int32_t>(pages_off);
    header_.dense_cta_off = static_cast<int32_t>(cta_off);
    header_.merge_indptr_off = static_cast<int32_t>(indptr_off);
    header_.merge_entries_off = static_cast<int32_t>(entries_off);
    header_.blob_words = static_cast<int32_t>(total);
    header_.num_segments = static_cast<int32_t>(segs.size());
    header_.max_page_id = -1;
    for (int32_t pg : pages_sec) header_.max_page_id = std::max(header_.max_page_id, pg);
    header_.unique_tokens = unique_tokens;
    header_.q_per_req = 1;
    header_.limits_off = any_limits ? static_cast<int32_t>(limits_off) : -1;
    header_.dense_q_off = static_cast<int32_t>(dense_q_off);
    header_.dense_q_width = static_cast<int32_t>(dense_q_width);
    for (GrowSlot& g : grow_)
        if (g.item >= 0) g.next_page += static_cast<int32_t>(pages_off);
    return 0;
}

int WorkList::can_advance(const std::vector<Growth>& growth) const {
    if (header_.q_per_req != 1) return 0;       // per-position limits are not patched in place
    if (grow_.empty()) return growth.empty() ? 1 : 0;
    for (const Growth& gr : growth) {
        if (gr.seq < 0 || gr.seq >= static_cast<int>(grow_.size())) return 0;
        const GrowSlot& g = grow_[gr.seq];
        if (g.item < 0 || gr.num_pages > g.slack) return 0;
        // the new tokens must fill the last page first and then exactly the appended pages
        const int room = header_.page_size - g.last_tokens;
        const int beyond = gr.tokens - room;
        const int need = beyond > 0 ? ceil_div(beyond, header_.page_size) : 0;
        if (need != gr.num_pages) return 0;
    }
    return 1;
}

void WorkList::advance(const std::vector<Growth>& growth) {
    for (const Growth& gr : growth) {
        GrowSlot& g = grow_[gr.seq];
        int32_t* item = blob_.data() + header_.items_off + static_cast<size_t>(g.item) * 8;
        item[3] += gr.tokens;                   // kv_len
        item[6] += gr.tokens;                   // cost
        for (int i = 0; i < gr.num_pages; ++i) {
            blob_[static_cast<size_t>(g.next_page) + i] = gr.pages[i];
            header_.max_page_id = std::max(header_.max_page_id, gr.pages[i]);
        }
        g.next_page += gr.num_pages;
        g.slack -= gr.num_pages;
        g.last_tokens = (g.last_tokens + gr.tokens - 1) % header_.page_size + 1;
        header_.unique_tokens += gr.tokens;
        header_.stream_tokens += gr.tokens;
        header_.stream_unique_tokens += gr.tokens;
    }
}

}  // namespace pat

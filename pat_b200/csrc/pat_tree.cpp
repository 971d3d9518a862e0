// Radix tree + plan packer; see pat_tree.h for the two semantics it can follow.
#include "pat_tree.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <map>

namespace pat {

namespace {

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Python's % for a possibly negative left operand.
inline long long py_mod(long long a, long long b) {
    long long r = a % b;
    return (r != 0 && ((r < 0) != (b < 0))) ? r + b : r;
}

// Padded-matmul cost model of the alternative heuristic
// (prefix_attn/prefix_tree.py:16-45).
inline long long cost_mm(long long nq, long long nk, long long hratio) {
    const long long tile = (nq * hratio >= 64) ? 64 : 16;
    const long long pad = tile - (py_mod(nq - 1, tile) + 1);
    return pad * nk * hratio;
}

}  // namespace

Tree::Tree(int block_size, Semantics sem) : block_size_(block_size), sem_(sem) {
    // kPython: add_node(-1) keeps the default s_value = 1 for the root
    // (prefix_tree.py:57,60); kCpp: the root starts at 0 (prefix_tree.h:74).
    add_node(-1, sem == Semantics::kPython ? 1 : 0, 0, {}, nullptr, 0);
}

int Tree::add_node(int parent, int s_value, int length, std::vector<int> seqs, const int* pages,
                   int num_pages) {
    nodes_.emplace_back();
    TreeNode& n = nodes_.back();
    n.parent = parent;
    n.s_value = s_value;
    n.length = length;
    n.seq_indices = std::move(seqs);
    n.pages = pages;
    n.num_pages = num_pages;
    return static_cast<int>(nodes_.size()) - 1;
}

int Tree::node_pages(const TreeNode& n) const {
    if (sem_ == Semantics::kPython) return n.num_pages;
    return n.pages ? ceil_div(n.length, block_size_) : 0;
}

std::vector<int> Tree::children_in_order(int node) const {
    const TreeNode& n = nodes_[node];
    std::vector<int> out;
    out.reserve(n.children.size());
    if (sem_ == Semantics::kPython) {
        for (int key : n.child_keys) out.push_back(n.children.at(key));
    } else {
        for (const auto& kv : n.children) out.push_back(kv.second);
    }
    return out;
}

void Tree::insert(int seq, int seq_len, const int* pages, int left) {
    const int bs = block_size_;
    int at = 0;
    while (left > 0) {
        const int head = pages[0];
        auto it = nodes_[at].children.find(head);
        if (it == nodes_[at].children.end()) {
            const int leaf = add_node(at, 1, seq_len, {seq}, pages, left);
            nodes_[at].children[head] = leaf;
            nodes_[at].child_keys.push_back(head);
            leaf_[seq] = leaf;
            return;
        }
        const int child = it->second;
        const int* edge = nodes_[child].pages;
        const int edge_n = node_pages(nodes_[child]);
        int shared = 0;
        if (sem_ == Semantics::kPython) {
            // bisection, as prefix_tree.py:81-89 (assumes agreement is a prefix)
            int lo = -1, hi = std::min(left, edge_n);
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (pages[mid] == edge[mid]) lo = mid; else hi = mid;
            }
            shared = lo + 1;
        } else {
            const int limit = std::min(edge_n, left);
            shared = static_cast<int>(std::mismatch(pages, pages + limit, edge).first - pages);
        }
        if (shared == edge_n) {
            nodes_[child].s_value += 1;
            nodes_[child].seq_indices.push_back(seq);
            at = child;
            left -= shared;
            seq_len -= shared * bs;
            pages += shared;
            continue;
        }
        // split the edge after `shared` pages
        const int split_key = edge[shared];
        const int edge_head = edge[0];
        std::vector<int> mid_seqs = nodes_[child].seq_indices;
        const int mid = add_node(at, nodes_[child].s_value + 1, shared * bs, std::move(mid_seqs), edge, shared);
        nodes_[mid].children[split_key] = child;
        nodes_[mid].child_keys.push_back(split_key);
        nodes_[at].children[edge_head] = mid;   // existing key: order unchanged
        nodes_[child].parent = mid;
        nodes_[child].pages = edge + shared;
        nodes_[child].num_pages -= shared;
        nodes_[child].length -= shared * bs;
        nodes_[mid].seq_indices.push_back(seq);
        if (shared != left) {
            const int* rest = pages + shared;
            int len;
            if (sem_ == Semantics::kPython) len = std::min(left * bs, seq_len) - shared * bs;
            else len = seq_len - shared * bs;
            const int leaf = add_node(mid, 1, len, {seq}, rest, left - shared);
            nodes_[mid].children[rest[0]] = leaf;
            nodes_[mid].child_keys.push_back(rest[0]);
            leaf_[seq] = leaf;
        } else {
            leaf_[seq] = mid;
        }
        return;
    }
    leaf_[seq] = at;
}

int Tree::build_padded(const int32_t* seq_lens, const int32_t* table, int num_seqs, int row_stride) {
    if (num_seqs < 0 || row_stride < 0 || (num_seqs > 0 && (!seq_lens || !table))) return kTreeBadArgument;
    // private copy so that nodes never point into caller memory
    size_t total = 0;
    std::vector<int> counts(num_seqs);
    for (int i = 0; i < num_seqs; ++i) {
        const int len = seq_lens[i];
        int c = len > 0 ? ceil_div(len, block_size_) : 0;
        if (c > row_stride) return kTreeBadArgument;
        counts[i] = c;
        total += c;
    }
    const size_t base = pool_.size();
    if (base != 0) return kTreeBadArgument;  // one build per tree object
    pool_.reserve(total);               // filled by appending: no zero-fill of a megabyte first
    size_t pos = 0;
    nodes_.reserve(static_cast<size_t>(num_seqs) * 2 + 1);
    std::vector<size_t> starts(num_seqs);
    for (int i = 0; i < num_seqs; ++i) {
        starts[i] = pos;
        const int32_t* row = table + static_cast<size_t>(i) * row_stride;
        pool_.insert(pool_.end(), row, row + counts[i]);
        pos += counts[i];
    }
    leaf_.assign(num_seqs, 0);
    seq_len_.assign(seq_lens, seq_lens + num_seqs);
    row_start_ = starts;
    row_pages_ = counts;
    grown_.assign(num_seqs, {});
    leaf_pages_.assign(num_seqs, {});
    for (int i = 0; i < num_seqs; ++i) insert(i, seq_lens[i], pool_.data() + starts[i], counts[i]);
    split_per_seq_.assign(num_seqs, 0);
    batch_ = num_seqs;
    built_ = true;
    return kTreeOk;
}

int Tree::build_ragged(const int32_t* seq_lens, const int32_t* flat, const int64_t* offsets, int num_seqs) {
    if (num_seqs < 0 || (num_seqs > 0 && (!seq_lens || !offsets))) return kTreeBadArgument;
    if (!pool_.empty()) return kTreeBadArgument;
    const int64_t total = num_seqs > 0 ? offsets[num_seqs] : 0;
    if (total < 0 || (total > 0 && !flat)) return kTreeBadArgument;
    pool_.assign(flat, flat + total);
    nodes_.reserve(static_cast<size_t>(num_seqs) * 2 + 1);
    leaf_.assign(num_seqs, 0);
    seq_len_.assign(seq_lens, seq_lens + num_seqs);
    row_start_.assign(num_seqs, 0);
    row_pages_.assign(num_seqs, 0);
    grown_.assign(num_seqs, {});
    leaf_pages_.assign(num_seqs, {});
    for (int i = 0; i < num_seqs; ++i) {
        const int64_t lo = offsets[i], hi = offsets[i + 1];
        if (lo < 0 || hi < lo || hi > total) return kTreeBadArgument;
        row_start_[i] = static_cast<size_t>(lo);
        row_pages_[i] = static_cast<int>(hi - lo);
        insert(i, seq_lens[i], pool_.data() + lo, static_cast<int>(hi - lo));
    }
    split_per_seq_.assign(num_seqs, 0);
    batch_ = num_seqs;
    built_ = true;
    return kTreeOk;
}

int Tree::plan_advance(const int32_t* seq_lens, const int32_t* table, int num_seqs, int row_stride,
                       std::vector<Growth>& out) const {
    out.clear();
    if (!built_ || num_seqs != batch_) return 0;
    if (num_seqs > 0 && (!seq_lens || !table)) return kTreeBadArgument;
    const int bs = block_size_;
    for (int i = 0; i < num_seqs; ++i) {
        const int old_len = seq_len_[i], new_len = seq_lens[i];
        if (new_len < old_len) return 0;
        const int old_np = old_len > 0 ? ceil_div(old_len, bs) : 0;
        const int new_np = new_len > 0 ? ceil_div(new_len, bs) : 0;
        if (new_np > row_stride) return kTreeBadArgument;
        // the part of the row the tree was built from (and has grown by since) must be unchanged
        const int32_t* row = table + static_cast<size_t>(i) * row_stride;
        const int built_np = std::min(row_pages_[i], old_np);
        if (built_np > 0 && std::memcmp(row, pool_.data() + row_start_[i], sizeof(int32_t) * built_np) != 0) return 0;
        const std::vector<int32_t>& g = grown_[i];
        if (built_np + static_cast<int>(g.size()) != old_np) return 0;
        if (!g.empty() && std::memcmp(row + built_np, g.data(), sizeof(int32_t) * g.size()) != 0) return 0;
        if (new_len == old_len) continue;
        // a request that grows must end in a leaf of its own whose edge ends with the request
        const TreeNode& leaf = nodes_[leaf_[i]];
        if (old_len <= 0 || row_pages_[i] > old_np || leaf_[i] == 0 || !leaf.children.empty() || leaf.s_value != 1 ||
            leaf.seq_indices.size() != 1 || leaf.seq_indices[0] != i)
            return 0;
        out.push_back(Growth{i, new_len - old_len, new_np - old_np, row + old_np});
    }
    return 1;
}

void Tree::apply_advance(const std::vector<Growth>& growth) {
    for (const Growth& g : growth) {
        TreeNode& leaf = nodes_[leaf_[g.seq]];
        if (g.num_pages > 0) {
            std::vector<int32_t>& buf = leaf_pages_[g.seq];
            const int have = node_pages(leaf);
            if (buf.empty()) {
                buf.reserve(static_cast<size_t>(have) + 64);
                buf.assign(leaf.pages, leaf.pages + have);
            }
            buf.insert(buf.end(), g.pages, g.pages + g.num_pages);
            leaf.pages = buf.data();
            leaf.num_pages = static_cast<int>(buf.size());
            grown_[g.seq].insert(grown_[g.seq].end(), g.pages, g.pages + g.num_pages);
        }
        leaf.length += g.tokens;
        seq_len_[g.seq] += g.tokens;
    }
    // a freshly built tree carries no plan
    buckets_.clear();
    std::fill(split_per_seq_.begin(), split_per_seq_.end(), 0);
    max_split_ = max_seqs_ = max_blocks_ = 0;
}

int Tree::emit(const std::vector<int>& queries, int begin, int count, int mm,
               const std::shared_ptr<const std::vector<int>>& pages, int kv_len, std::vector<Box>& out) {
    (void)begin;
    const int have = static_cast<int>(queries.size());
    for (int s = 0; s < count; s += mm) {
        Box box;
        const int lo = std::min(s, have);
        const int hi = std::min(std::min(s + mm, count), have);
        box.q_table.assign(queries.begin() + lo, queries.begin() + hi);
        box.pages = pages;
        box.page_lo = 0;
        box.page_hi = static_cast<int>(pages->size());
        box.kv_len = kv_len;
        if (sem_ == Semantics::kPython) {
            box.num_seqs = std::min(mm, count - s);
            if (box.q_table.empty()) return kTreeEmptyQueryBox;
        } else {
            box.num_seqs = static_cast<int>(box.q_table.size());
        }
        if (!box.q_table.empty()) {
            box.rank = split_per_seq_[box.q_table[0]];
            for (int q : box.q_table) split_per_seq_[q] += 1;
        }
        out.push_back(std::move(box));
    }
    return kTreeOk;
}

int Tree::walk(int node, int mm, int hratio, bool cost_model, const std::vector<int>& inherited,
               std::vector<Box>& out) {
    const int n_pages = node_pages(nodes_[node]);
    auto here = std::make_shared<std::vector<int>>(inherited);
    if (nodes_[node].pages) here->insert(here->end(), nodes_[node].pages, nodes_[node].pages + n_pages);
    const int kv_len = block_size_ * static_cast<int>(inherited.size()) + nodes_[node].length;

    if (nodes_[node].children.empty()) {
        return emit(nodes_[node].seq_indices, 0, nodes_[node].s_value, mm, here, kv_len, out);
    }

    const std::vector<int> kids = children_in_order(node);
    int remaining = nodes_[node].s_value;
    std::vector<int> folded, separate;
    for (int child : kids) {
        const int sc = nodes_[child].s_value;
        bool fold;
        if (cost_model) {
            const long long S = remaining, lc = nodes_[child].length, kv = kv_len, hr = hratio;
            // SplitK: this node once for all S, child alone, plus the reduction
            const double split_k = static_cast<double>(cost_mm(S, lc, hr) + cost_mm(sc, kv, hr)) +
                                   0.1 * static_cast<double>(sc) * static_cast<double>(hr);
            // SplitQ: the child carries this node's KV with it
            const double split_q = static_cast<double>(cost_mm(S - sc, kv, hr) + cost_mm(sc, kv + lc, hr));
            fold = split_k > split_q;
        } else if (remaining == sc) {
            fold = true;
        } else {
            const long long saved = static_cast<long long>(ceil_div(remaining, mm)) -
                                    ceil_div(remaining - sc, mm) - ceil_div(sc, mm);
            fold = saved * kv_len + 4LL * sc >= 0;
        }
        if (fold) {
            remaining -= sc;
            folded.push_back(child);
        } else {
            separate.push_back(child);
        }
    }

    if (remaining != 0) {
        std::vector<int> queries;
        int count;
        if (sem_ == Semantics::kPython) {
            for (int child : separate)
                queries.insert(queries.end(), nodes_[child].seq_indices.begin(), nodes_[child].seq_indices.end());
            count = remaining;
        } else {
            std::vector<uint8_t> gone(split_per_seq_.size(), 0);
            for (int child : folded)
                for (int q : nodes_[child].seq_indices) gone[q] = 1;
            queries.reserve(nodes_[node].s_value);
            for (int q : nodes_[node].seq_indices)
                if (!gone[q]) queries.push_back(q);
            count = static_cast<int>(queries.size());
        }
        const int rc = emit(queries, 0, count, mm, here, kv_len, out);
        if (rc != kTreeOk) return rc;
    }

    for (int child : separate) {
        const int rc = walk(child, mm, hratio, cost_model, {}, out);
        if (rc != kTreeOk) return rc;
    }
    for (int child : folded) {
        const int rc = walk(child, mm, hratio, cost_model, *here, out);
        if (rc != kTreeOk) return rc;
    }
    return kTreeOk;
}

int Tree::balance(std::vector<Box>& boxes, int kv_heads) {
    if (boxes.empty()) return kTreeOk;
    const int bs = block_size_;
    const bool py = sem_ == Semantics::kPython;

    auto piece = [](const Box& src, int lo, int hi, int kv, int rank) {
        Box b;
        b.q_table = src.q_table;
        b.pages = src.pages;
        b.page_lo = lo;
        b.page_hi = hi;
        b.num_seqs = src.num_seqs;
        b.kv_len = kv;
        b.rank = rank;
        return b;
    };

    // phase 1: crop boxes far longer than the average long box
    long long total_pages = 0;
    int long_boxes = 0;
    for (const Box& b : boxes) {
        if (py ? (b.kv_len > 256) : (b.kv_len >= 128)) {
            total_pages += b.num_pages();
            ++long_boxes;
        }
    }
    std::vector<Box> cropped;
    cropped.reserve(boxes.size() * 2);
    if (long_boxes != 0) {
        const double average = static_cast<double>(total_pages) / long_boxes;
        const double limit = average * 5.0;
        for (Box& box : boxes) {
            const int n = box.num_pages();
            if (!(static_cast<double>(n) > limit)) {
                cropped.push_back(std::move(box));
                continue;
            }
            int parts, step;
            if (py) {
                parts = static_cast<int>(std::ceil(static_cast<double>(n) / average));
                step = static_cast<int>(std::ceil(static_cast<double>(n) / static_cast<double>(parts)));
            } else {
                parts = ceil_div(n, static_cast<int>(average));
                step = ceil_div(n, parts);
            }
            for (int i = 0; i < parts; ++i) {
                int lo = i * step;
                int hi = std::min((i + 1) * step, n);
                if (!py && lo >= hi) break;
                if (py && hi < lo) hi = lo;  // empty Python slice
                if (py && lo > n) lo = hi = n;
                const int kv = std::min(box.kv_len - i * step * bs, step * bs);
                int rank = box.rank;
                if (i != 0) {
                    if (box.q_table.empty()) {
                        if (py) return kTreeEmptyQueryBox;
                        rank = 0;
                    } else {
                        rank = split_per_seq_[box.q_table[0]];
                        for (int q : box.q_table) split_per_seq_[q] += 1;
                    }
                }
                cropped.push_back(piece(box, box.page_lo + lo, box.page_lo + hi, kv, rank));
            }
        }
    } else {
        cropped = std::move(boxes);
    }

    // phase 2: halve the longest box until there are enough boxes
    int want;
    if (kv_heads <= 4) want = 54;
    else if (kv_heads <= 8) want = 27;
    else if (kv_heads <= 16) want = 13;
    else if (kv_heads <= 32) want = 6;
    else want = 4;

    auto max_split = [&]() {
        int m = py ? INT32_MIN : 0;
        for (int v : split_per_seq_) m = std::max(m, v);
        return m;
    };

    if (static_cast<int>(cropped.size()) < want) {
        while (static_cast<int>(cropped.size()) < want && max_split() < 32) {
            int pick = -1;
            int longest = py ? -1 : 0;
            for (size_t i = 0; i < cropped.size(); ++i) {
                if (cropped[i].num_pages() > longest) {
                    longest = cropped[i].num_pages();
                    pick = static_cast<int>(i);
                }
            }
            if (pick < 0) break;
            Box box = std::move(cropped[pick]);
            if (py) {
                cropped.erase(cropped.begin() + pick);
            } else {
                if (pick != static_cast<int>(cropped.size()) - 1) cropped[pick] = std::move(cropped.back());
                cropped.pop_back();
            }
            const int n = box.num_pages();
            if (py ? (n <= 8) : (n < 8)) {
                cropped.push_back(std::move(box));
                break;
            }
            if (box.q_table.empty()) return kTreeEmptyQueryBox;
            const int half = ceil_div(n, 2);
            Box first = piece(box, box.page_lo, box.page_lo + half, std::min(box.kv_len, half * bs), box.rank);
            Box second = piece(box, box.page_lo + half, box.page_hi,
                               std::min(box.kv_len - half * bs, (n - half) * bs),
                               split_per_seq_[box.q_table[0]]);
            for (int q : first.q_table) split_per_seq_[q] += 1;
            cropped.push_back(std::move(first));
            cropped.push_back(std::move(second));
        }
    }
    boxes = std::move(cropped);
    return kTreeOk;
}

void Tree::mnw_of(int rows, int kv_len, int out[3]) const {
    int m = 16, w = 1;
    if (rows > 32) { m = 64; w = 4; }
    else if (rows > 16) { m = 32; w = 2; }
    int n;
    if (kv_len < 32) n = 16;
    else if (kv_len < 64) n = 32;
    else if (sem_ == Semantics::kPython ? (kv_len <= 128) : (kv_len < 128)) n = 64;
    else n = 128;
    if (m == 64) n = std::max(32, n);
    out[0] = m; out[1] = n; out[2] = w;
}

int Tree::pack(const int32_t* mnws, int num_mnws, int hratio, int kv_heads, bool use_compute_model) {
    if (!built_) return kTreeNotBuilt;
    if (hratio <= 0 || num_mnws < 0 || (num_mnws > 0 && !mnws)) return kTreeBadArgument;
    static const int kDefault[11][3] = {
        {64, 128, 4}, {64, 64, 4}, {64, 32, 4},
        {32, 128, 2}, {32, 64, 2}, {32, 32, 2}, {32, 16, 2},
        {16, 128, 1}, {16, 64, 1}, {16, 32, 1}, {16, 16, 1}};
    std::vector<std::vector<int>> shapes;
    if (num_mnws == 0) {
        for (const auto& s : kDefault) shapes.push_back({s[0], s[1], s[2]});
    } else {
        for (int i = 0; i < num_mnws; ++i) shapes.push_back({mnws[3 * i], mnws[3 * i + 1], mnws[3 * i + 2]});
    }
    int max_m = 0;
    for (const auto& s : shapes) max_m = std::max(max_m, s[0]);
    int mm = max_m / hratio;
    const bool py = sem_ == Semantics::kPython;
    if (mm < 1) {
        if (py) {
            // range(0, S, 0) raises in Python unless there is nothing to walk
            if (!nodes_[0].children.empty()) return kTreeZeroQueriesPerBox;
        }
        mm = 1;
    }

    std::vector<Box> boxes;
    const bool cost_model = py && use_compute_model;
    for (int child : children_in_order(0)) {
        const int rc = walk(child, mm, hratio, cost_model, {}, boxes);
        if (rc != kTreeOk) return rc;
    }
    {
        const int rc = balance(boxes, kv_heads);
        if (rc != kTreeOk) return rc;
    }

    std::map<std::vector<int>, std::vector<const Box*>> grouped;
    for (const auto& s : shapes) grouped[s];
    if (shapes.size() == 1) {
        auto& g = grouped[shapes[0]];
        for (const Box& b : boxes) g.push_back(&b);
    } else {
        for (const Box& b : boxes) {
            int t[3];
            mnw_of(static_cast<int>(b.q_table.size()) * hratio, b.kv_len, t);
            auto it = grouped.find({t[0], t[1], t[2]});
            if (it == grouped.end()) {
                if (py) return kTreeUnknownBucket;
                it = grouped.find(shapes[0]);
            }
            it->second.push_back(&b);
        }
    }

    if (py) {
        buckets_.clear();
        max_seqs_ = 0;
        max_blocks_ = 0;
    }
    for (const auto& s : shapes) {
        const auto& group = grouped[s];
        if (group.empty()) continue;
        Bucket bk;
        bk.mnw[0] = s[0]; bk.mnw[1] = s[1]; bk.mnw[2] = s[2];
        bk.ctas = static_cast<int>(group.size());
        for (const Box* b : group) {
            bk.max_seqs = std::max(bk.max_seqs, static_cast<int>(b->q_table.size()));
            bk.max_blocks = std::max(bk.max_blocks, b->num_pages());
        }
        bk.q_table.assign(static_cast<size_t>(bk.ctas) * bk.max_seqs, 0);
        bk.block_table.assign(static_cast<size_t>(bk.ctas) * bk.max_blocks, 0);
        bk.num_seqs.reserve(bk.ctas);
        bk.ranks.reserve(bk.ctas);
        bk.kv_lens.reserve(bk.ctas);
        for (int i = 0; i < bk.ctas; ++i) {
            const Box* b = group[i];
            std::copy(b->q_table.begin(), b->q_table.end(), bk.q_table.begin() + static_cast<size_t>(i) * bk.max_seqs);
            std::copy(b->pages->begin() + b->page_lo, b->pages->begin() + b->page_hi,
                      bk.block_table.begin() + static_cast<size_t>(i) * bk.max_blocks);
            bk.num_seqs.push_back(b->num_seqs);
            bk.ranks.push_back(b->rank);
            bk.kv_lens.push_back(b->kv_len);
        }
        max_seqs_ = std::max(max_seqs_, bk.max_seqs);
        max_blocks_ = std::max(max_blocks_, bk.max_blocks);
        buckets_.push_back(std::move(bk));
    }
    max_split_ = 0;
    if (py && !split_per_seq_.empty()) max_split_ = INT32_MIN;
    for (int v : split_per_seq_) max_split_ = std::max(max_split_, v);
    return kTreeOk;
}

}  // namespace pat

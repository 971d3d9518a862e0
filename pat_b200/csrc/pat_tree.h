// Native radix tree over physical page ids + tile-plan packer (host only).
//
// Replaces the reference's header-only scheduler csrc/prefix_tree.h
// (PrefixTree::build_radix_tree :84-181, pack_schedule :183-324,
// _tree_heuristics :347-479, balancePack :481-621, getMNW :330-345) and is also
// able to reproduce the pure-Python scheduler prefix_attn/prefix_tree.py bit for
// bit.  The two reference schedulers disagree in a dozen details (thresholds,
// iteration order, how the queries left at an inner node are collected); the
// `Semantics` switch selects which one is followed:
//
//   kPython : prefix_tree.py  (children in insertion order, getMNW maps 128
//             tokens to N=64, crop population kv > 256, float ceil, stop at
//             <= 8 pages, pop/append order, cost model honoured)
//   kCpp    : prefix_tree.h   (children in std::unordered_map order, 128 tokens
//             -> N=128, population kv >= 128, integer ceil, stop at < 8 pages,
//             swap-with-back order, cost model ignored, plans accumulate over
//             repeated pack calls)
//
// No torch, no CUDA: plain C++17.
#pragma once

#include <cstdint>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

namespace pat {

enum class Semantics : int { kPython = 0, kCpp = 1 };

struct TreeNode {
    int parent = -1;
    int s_value = 0;            // requests passing through this node
    int length = 0;             // valid tokens on the edge into this node
    const int* pages = nullptr; // first page id of the edge (points into Tree::pool_)
    int num_pages = 0;          // kPython: explicit; kCpp: derived from length
    std::vector<int> seq_indices;
    std::unordered_map<int, int> children;  // first page id -> child (lookup + kCpp order)
    std::vector<int> child_keys;             // keys in insertion order (kPython order)
};

struct Box {
    std::vector<int> q_table;
    std::shared_ptr<const std::vector<int>> pages;  // full list; [page_lo, page_hi) is this box's
    int page_lo = 0, page_hi = 0;
    int num_seqs = 0;
    int kv_len = 0;
    int rank = 0;
    int num_pages() const { return page_hi - page_lo; }
};

struct Bucket {
    int mnw[3] = {0, 0, 0};
    int ctas = 0;
    int max_seqs = 0;
    int max_blocks = 0;
    std::vector<int32_t> q_table;      // [ctas, max_seqs], 0-padded
    std::vector<int32_t> block_table;  // [ctas, max_blocks], 0-padded
    std::vector<int32_t> num_seqs;     // [ctas]
    std::vector<int32_t> ranks;        // [ctas]
    std::vector<int32_t> kv_lens;      // [ctas]
};

// Growth of one request between two decode steps (Tree::plan_advance).
struct Growth {
    int seq;
    int tokens;                 // new valid tokens at the end of the request
    int num_pages;              // pages appended to its table row
    const int32_t* pages;       // points into the caller's table
};

enum TreeStatus : int {
    kTreeOk = 0,
    kTreeBadArgument = -1,
    kTreeEmptyQueryBox = -2,   // a box with no query (Python raises IndexError there)
    kTreeZeroQueriesPerBox = -3,  // max M < HRatio under Python semantics (range() step 0)
    kTreeUnknownBucket = -4,   // Python raises KeyError for a tile shape outside MNWs
    kTreeNotBuilt = -5,
};

class Tree {
public:
    Tree(int block_size, Semantics sem);

    // Padded table [num_seqs, row_stride]; each row is cut to ceil(len/block) pages.
    int build_padded(const int32_t* seq_lens, const int32_t* table, int num_seqs, int row_stride);
    // Ragged page lists: row i is flat[offsets[i] .. offsets[i+1]).
    int build_ragged(const int32_t* seq_lens, const int32_t* flat, const int64_t* offsets, int num_seqs);

    int pack(const int32_t* mnws, int num_mnws, int hratio, int kv_heads, bool use_compute_model);

    // --- in-place growth between decode steps ------------------------------------
    // A decode step appends tokens (and now and then a page) to requests whose tables are
    // otherwise unchanged.  When every request ends in a leaf that belongs to it alone, the tree
    // a fresh build would produce from the new tables is this tree with longer leaf edges.
    // plan_advance checks that (same batch, no request shrinks, the old part of every row
    // unchanged, every growing request alone in its leaf) and lists the growth; it returns 1
    // when the tree can grow in place, 0 when it has to be rebuilt, < 0 on a bad argument, and
    // changes nothing.  apply_advance performs the growth and forgets the packed plan (a fresh
    // tree has none).
    int plan_advance(const int32_t* seq_lens, const int32_t* table, int num_seqs, int row_stride,
                     std::vector<Growth>& out) const;
    void apply_advance(const std::vector<Growth>& growth);
    int leaf_of(int seq) const { return leaf_[seq]; }
    int seq_len(int seq) const { return seq_len_[seq]; }

    // --- results -------------------------------------------------------------
    const std::vector<Bucket>& buckets() const { return buckets_; }
    const std::vector<int32_t>& split_per_seq() const { return split_per_seq_; }
    int max_split_per_seq() const { return max_split_; }
    int max_seqs_in_cta() const { return max_seqs_; }
    int max_blocks_in_cta() const { return max_blocks_; }
    int batch() const { return batch_; }
    int block_size() const { return block_size_; }
    Semantics semantics() const { return sem_; }

    // --- tree inspection (tests) --------------------------------------------
    const std::vector<TreeNode>& nodes() const { return nodes_; }
    std::vector<int> children_in_order(int node) const;

private:
    int add_node(int parent, int s_value, int length, std::vector<int> seqs, const int* pages, int num_pages);
    void insert(int seq, int seq_len, const int* pages, int num_pages);
    int node_pages(const TreeNode& n) const;
    int walk(int node, int mm, int hratio, bool cost_model, const std::vector<int>& inherited,
             std::vector<Box>& out);
    int emit(const std::vector<int>& queries, int begin, int count, int mm,
             const std::shared_ptr<const std::vector<int>>& pages, int kv_len, std::vector<Box>& out);
    int balance(std::vector<Box>& boxes, int kv_heads);
    void mnw_of(int rows, int kv_len, int out[3]) const;

    int block_size_;
    Semantics sem_;
    int batch_ = 0;
    bool built_ = false;
    std::vector<int32_t> pool_;   // private copy of every page list
    std::vector<int> leaf_;       // node in which each request ends
    std::vector<int32_t> seq_len_;
    std::vector<size_t> row_start_;             // each request's row in pool_ (as built)
    std::vector<int> row_pages_;                // pages of that row
    std::vector<std::vector<int32_t>> grown_;   // pages appended to a request since the build
    std::vector<std::vector<int32_t>> leaf_pages_;  // a grown leaf's page list (the node points here)
    std::vector<TreeNode> nodes_;
    std::vector<int32_t> split_per_seq_;
    std::vector<Bucket> buckets_;
    int max_split_ = 0, max_seqs_ = 0, max_blocks_ = 0;
};

}  // namespace pat

// Work-list builder (host only): reference-format plan -> device work items.
//
// A reference plan (csrc/prefix_tree.h:7-25 / prefix_attn/data_class.py:173-207)
// is a set of boxes "queries q_table[:n] x all their heads attend to the first
// kv_in_CTA tokens of these pages".  The reference runs one CTA per box
// (csrc/pat_fwd_launch_template.h:35-50) and labels each box's partial result
// with one CTA_rank (csrc/block_info.h:28-35), which can collide.  This builder
// keeps the plan's meaning and re-derives the execution:
//
//   1. boxes with the same page list are fused; pages are then regrouped by the
//      set of fused boxes that contain them, so that every (page, valid tokens)
//      pair is attended by all its queries in ONE segment and is read from HBM
//      once (attention is invariant to KV order, so regrouping is exact);
//   2. segments with few query rows become streaming items (<= 16 rows x one KV
//      chunk, run for every KV head), ordered longest first;
//   3. segments shared by many rows become dense items for the tensor-core
//      kernel: per KV head, the token ranges of all (segment, <= 256 rows) units
//      are laid end to end and cut into equal shares, one share per persistent
//      CTA, so that every CTA streams the same number of tokens;
//   4. every (item, query, KV head) triple owns a private partial slot ("entry":
//      hratio rows of D floats + LSEs), and a CSR list per (request, KV head)
//      tells the merge kernel which entries to combine.
//
// Multiplicity is preserved: a query that attends a page twice in the plan
// attends it twice here.
#pragma once

#include <cstdint>
#include <vector>

#include "pat_tree.h"

namespace pat {

struct PlanBucketView {
    int ctas;
    const int32_t* q_table;      // [ctas, q_stride]
    int q_stride;
    const int32_t* block_table;  // [ctas, block_stride]
    int block_stride;
    const int32_t* num_seqs;     // [ctas]
    const int32_t* kv_lens;      // [ctas]
};

struct WorkOptions {
    int num_sms = 148;
    int stream_rows = 16;              // query rows per streaming item
    int dense_rows = 128;              // query rows per dense item (0 = dense kernel off)
    int dense_min_rows = 17;           // segments with at least this many rows go to the dense kernel
    int chunk_tokens_min = 256;
    int chunk_tokens_max = 2048;
    // A dense share is not cut (much) below this many tokens.  Two tiles: with 512 a rank of a 4-
    // or 8-GPU run on a short batch left most SMs without dense work (22.7 vs 26.0 us per step on
    // one rank of four of the two-level tree); with 128 the extra partial rows cost the merge more
    // than the dense kernel gains.
    int dense_piece_tokens_min = 256;
    int items_per_sm = 4;              // target number of streaming items per SM (all KV heads)
    // Estimated time of one 128-token tile of the dense kernel.  When a work list has streaming
    // work too, the dense kernel runs beside the streaming kernel and gets only as many CTAs as
    // keep its estimated time well below the estimated time of the whole step.
    // < 0: the dense kernel is cut for every SM.
    int dense_tile_ns = 1200;
    // Pages of slack behind the page list of a segment that one request owns alone (only in
    // lists built straight from a tree): room for WorkList::advance to append pages in place.
    int grow_slack_pages = 8;
};

// One work item = 8 int32 on the device.
struct WorkItem {
    int32_t q_off;       // offset of its query ids in the query section
    int32_t nq;          // number of queries (rows = nq * hratio)
    int32_t page_off;    // offset of its first page id in the page section
    int32_t kv_len;      // valid tokens (the first kv_len tokens of its pages)
    int32_t entry_base;  // streaming: entry of (query i, head h) = entry_base + i * kv_heads + h
                         // dense:     entry of query i            = entry_base + i
    int32_t kv_head;     // dense items: the KV head; streaming items: -1 (run for every head)
    int32_t cost;        // tokens (ordering key)
    int32_t tok_lo;      // first token of the item inside its segment (used with the per-query limits)
};
static_assert(sizeof(WorkItem) == 32, "device layout");

struct WorkHeader {
    int32_t batch;
    int32_t hratio;
    int32_t page_size;
    int32_t kv_heads;
    int32_t num_stream_items;     // items [0, num_stream_items), longest first
    int32_t num_dense_items;      // then the dense items, grouped by CTA
    int32_t num_dense_ctas;       // persistent CTAs of the dense kernel
    int32_t num_entries;
    int32_t max_entries_per_list;
    int32_t items_off;            // all offsets in int32 units from the start of the blob
    int32_t queries_off;
    int32_t pages_off;
    int32_t dense_cta_off;        // [num_dense_ctas + 1] first dense item of each CTA
    int32_t merge_indptr_off;     // [batch * kv_heads + 1]
    int32_t merge_entries_off;    // [sum of list lengths]
    int32_t blob_words;
    int32_t num_segments;
    int32_t max_page_id;          // largest page id any item touches (-1 if none)
    int64_t unique_tokens;        // sum of segment tokens (each page counted once)
    int64_t stream_tokens;        // tokens read by streaming items per KV head (a segment counts once per row chunk)
    int64_t dense_tokens;         // same for dense items
    int64_t stream_unique_tokens; // unique tokens of the segments the streaming kernel handles
    int64_t dense_unique_tokens;
    // Several query tokens per request (seqlen_q = q_per_req > 1): a "query" of the list is then the
    // pair (request, position), id = request * q_per_req + position, `batch` counts those pairs,
    // and the section at limits_off (parallel to the query section) holds, per (segment, query),
    // how many of the segment's tokens that position may see.  limits_off = -1 when every query
    // sees all tokens of its segments (q_per_req = 1).
    int32_t q_per_req;
    int32_t limits_off;
    // Query ids of the dense items as a table with a fixed row width (dense_rows / hratio ids per
    // item, -1 past an item's queries): the dense kernel fetches an item's ids without first
    // having read the item's record.
    int32_t dense_q_off;
    int32_t dense_q_width;
};

// A set of pages attended by the same queries (host-side intermediate of the builders).
struct WorkSegment {
    std::vector<int32_t> queries;
    std::vector<int32_t> pages;
    int64_t tokens = 0;
    int partial_tokens = 0;  // valid tokens of the (single, last) partial page, 0 if none
    int32_t q_off = 0, page_off = 0;
    int owner = -1;          // the one request that ends in this segment and may extend it, or -1
    std::vector<int32_t> limits;  // per query: visible tokens of this segment; empty = all of them
};

class WorkList {
public:
    // From a reference-format plan.  Returns 0 or a negative error (bad index / bad argument).
    int build(const PlanBucketView* buckets, int num_buckets, int batch, int hratio, int kv_heads,
              int page_size, int64_t num_cache_pages, const WorkOptions& opt);
    // Straight from a built radix tree: every edge of the tree is a segment (its pages, attended
    // by the requests that pass through it).  For every batch a block-id radix tree can express
    // this is the list `build` derives from the tree's packed plan - the plan's boxes are
    // regrouped into exactly these page sets - without packing the plan first, and it can be
    // advanced in place afterwards.
    // q_per_req > 1: every request carries that many query tokens, the last q_per_req tokens of
    // its context; position t attends to the first seq_len - q_per_req + 1 + t tokens.
    int build_from_tree(const Tree& tree, int hratio, int kv_heads, int64_t num_cache_pages,
                        const WorkOptions& opt, int q_per_req = 1);
    // After Tree::plan_advance said yes: 1 if the growth fits the slack of the owners' segments
    // (nothing is changed by the check), else 0.
    int can_advance(const std::vector<Growth>& growth) const;
    // Applies the growth to the blob and the header in place (item lengths, appended page ids).
    void advance(const std::vector<Growth>& growth);
    const WorkHeader& header() const { return header_; }
    const std::vector<int32_t>& blob() const { return blob_; }

private:
    int finish(std::vector<WorkSegment>& segs, int batch, int hratio, int kv_heads, int page_size,
               const WorkOptions& opt);
    struct GrowSlot {
        int32_t item = -1;       // streaming item (index in the blob) that holds the request's last tokens
        int32_t next_page = 0;   // blob index of the first free slot behind the segment's page list
        int32_t slack = 0;       // free slots left
        int32_t last_tokens = 0; // valid tokens in the segment's last page
    };
    WorkHeader header_{};
    std::vector<int32_t> blob_;
    std::vector<GrowSlot> grow_;  // per request; empty for lists built from a plan
};

}  // namespace pat

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
//   2. a segment becomes work items: query-row chunks (<= 16 rows for the
//      streaming kernel, <= 128/256 rows for the dense tensor-core kernel) times
//      KV chunks sized for load balance, ordered longest first;
//   3. every (item, query) pair owns a private partial slot ("entry"), and a
//      CSR list per query tells the merge kernel which entries to combine.
//
// Multiplicity is preserved: a query that attends a page twice in the plan
// attends it twice here.
#pragma once

#include <cstdint>
#include <vector>

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
    int stream_rows = 16;          // query rows per streaming item
    int dense_rows = 0;            // query rows per dense item (0 = dense kernel off)
    int dense_min_rows = 1 << 30;  // segments with at least this many rows go to the dense kernel
    int chunk_tokens_min = 256;
    int chunk_tokens_max = 2048;
    int dense_chunk_tokens_max = 2048;
    int items_per_sm = 8;          // target number of streaming items per SM (all KV heads)
    int fold_tokens = 0;           // shared segments with <= this many tokens are copied into each query
};

// One work item = 8 int32 on the device.
struct WorkItem {
    int32_t q_off;       // offset of its query ids in the query section
    int32_t nq;          // number of queries (rows = nq * hratio)
    int32_t page_off;    // offset of its first page id in the page section
    int32_t kv_len;      // valid tokens (the first kv_len tokens of its pages)
    int32_t entry_base;  // partial slot of its first query; slot of query i is entry_base + i
    int32_t kind;        // 0 = streaming, 1 = dense
    int32_t cost;        // tokens x row tiles (ordering key)
    int32_t reserved;
};
static_assert(sizeof(WorkItem) == 32, "device layout");

struct WorkHeader {
    int32_t batch;
    int32_t hratio;
    int32_t page_size;
    int32_t num_stream_items;   // items [0, num_stream_items) are streaming, longest first
    int32_t num_dense_items;    // then the dense items, longest first
    int32_t num_entries;
    int32_t max_entries_per_query;
    int32_t items_off;          // all offsets in int32 units from the start of the blob
    int32_t queries_off;
    int32_t pages_off;
    int32_t merge_indptr_off;   // [batch + 1]
    int32_t merge_entries_off;  // [num_entries]
    int32_t blob_words;
    int32_t num_segments;
    int32_t max_page_id;        // largest page id any item touches (-1 if none)
    int32_t reserved;
    int64_t unique_tokens;      // sum of segment tokens (each page counted once)
    int64_t stream_tokens;      // tokens read by streaming items (x row chunks)
    int64_t dense_tokens;
    int64_t stream_unique_tokens;
    int64_t dense_unique_tokens;
};

class WorkList {
public:
    // Returns 0 or a negative error (bad index / bad argument).
    int build(const PlanBucketView* buckets, int num_buckets, int batch, int hratio, int kv_heads,
              int page_size, int64_t num_cache_pages, const WorkOptions& opt);
    const WorkHeader& header() const { return header_; }
    const std::vector<int32_t>& blob() const { return blob_; }

private:
    WorkHeader header_{};
    std::vector<int32_t> blob_;
};

}  // namespace pat

// C ABI over the host-side scheduler and work-list builder (see include/pat_b200.h).
#include "../../include/pat_b200.h"

#include <new>
#include <vector>

#include "pat_tree.h"
#include "pat_work.h"

struct pat_tree {
    pat::Tree tree;
    pat_tree(int bs, pat::Semantics s) : tree(bs, s) {}
};

struct pat_work {
    pat::WorkList list;
};

namespace {

pat::WorkOptions to_options(const pat_work_options* o) {
    pat::WorkOptions w;
    // Defaults: query-row tiles of 16 through the streaming kernel; segments with
    // more than 16 rows go through the dense (tensor-core tile) kernel in tiles of
    // up to 128 rows.
    w.dense_rows = 128;
    w.dense_min_rows = 17;
    if (!o) return w;
    if (o->num_sms > 0) w.num_sms = o->num_sms;
    if (o->dense_min_rows > 0) w.dense_min_rows = o->dense_min_rows;
    if (o->chunk_tokens_min > 0) w.chunk_tokens_min = o->chunk_tokens_min;
    if (o->chunk_tokens_max > 0) w.chunk_tokens_max = o->chunk_tokens_max;
    if (o->dense_piece_tokens_min > 0) w.dense_piece_tokens_min = o->dense_piece_tokens_min;
    if (o->items_per_sm > 0) w.items_per_sm = o->items_per_sm;
    if (o->dense_tile_ns != 0) w.dense_tile_ns = o->dense_tile_ns;
    if (o->grow_slack_pages > 0) w.grow_slack_pages = o->grow_slack_pages;
    if (o->grow_slack_pages < 0) w.grow_slack_pages = 0;
    if (o->disable_dense) { w.dense_rows = 0; w.dense_min_rows = 1 << 30; }
    return w;
}

int map_work_error(int rc) { return rc == 0 ? PAT_OK : (rc == -1 ? PAT_ERR_BAD_ARGUMENT : PAT_ERR_BAD_PLAN); }

void copy_header(const pat::WorkHeader& h, pat_work_header* out) {
    out->batch = h.batch; out->hratio = h.hratio; out->page_size = h.page_size; out->kv_heads = h.kv_heads;
    out->num_stream_items = h.num_stream_items; out->num_dense_items = h.num_dense_items;
    out->num_dense_ctas = h.num_dense_ctas;
    out->num_entries = h.num_entries; out->max_entries_per_list = h.max_entries_per_list;
    out->items_off = h.items_off; out->queries_off = h.queries_off; out->pages_off = h.pages_off;
    out->dense_cta_off = h.dense_cta_off;
    out->merge_indptr_off = h.merge_indptr_off; out->merge_entries_off = h.merge_entries_off;
    out->blob_words = h.blob_words; out->num_segments = h.num_segments; out->max_page_id = h.max_page_id;
    out->unique_tokens = h.unique_tokens; out->stream_tokens = h.stream_tokens;
    out->dense_tokens = h.dense_tokens;
    out->stream_unique_tokens = h.stream_unique_tokens;
    out->dense_unique_tokens = h.dense_unique_tokens;
    out->q_per_req = h.q_per_req;
    out->limits_off = h.limits_off;
    out->dense_q_off = h.dense_q_off;
    out->dense_q_width = h.dense_q_width;
}

}  // namespace

extern "C" {

int pat_b200_abi_version(void) { return 4; }

const char* pat_b200_strerror(int status) {
    switch (status) {
        case PAT_OK: return "ok";
        case PAT_ERR_BAD_ARGUMENT: return "bad argument";
        case PAT_ERR_EMPTY_QUERY_BOX: return "list index out of range (a box has no query)";
        case PAT_ERR_ZERO_QUERIES_PER_BOX: return "range() arg 3 must not be zero (max tile M < HRatio)";
        case PAT_ERR_UNKNOWN_BUCKET: return "tile shape of a box is not in MNWs";
        case PAT_ERR_NOT_BUILT: return "build_radix_tree must be called before pack_schedule";
        case PAT_ERR_BAD_PLAN: return "plan tables are inconsistent (index out of range)";
        case PAT_ERR_UNSUPPORTED: return "unsupported dtype, head size, head ratio, page size or alignment";
        case PAT_ERR_WORKSPACE: return "workspace missing or too small";
        case PAT_ERR_CUDA: return "a CUDA call failed";
        case PAT_ERR_NO_DEVICE_CODE: return "this library only carries sm_100a device code";
        case PAT_ERR_TOO_LARGE: return "size exceeds a fixed limit";
        case PAT_ERR_NO_MEMORY: return "out of host memory";
        default: return "unknown status";
    }
}

pat_tree* pat_tree_create(int block_size, int semantics) {
    if (block_size <= 0 || (semantics != PAT_SEMANTICS_PYTHON && semantics != PAT_SEMANTICS_CPP)) return nullptr;
    return new (std::nothrow) pat_tree(block_size, static_cast<pat::Semantics>(semantics));
}

void pat_tree_destroy(pat_tree* t) { delete t; }

int pat_tree_build(pat_tree* t, const int32_t* seq_lens, const int32_t* block_table, int num_seqs,
                   int row_stride) {
    if (!t) return PAT_ERR_BAD_ARGUMENT;
    try {
        return t->tree.build_padded(seq_lens, block_table, num_seqs, row_stride);
    } catch (...) { return PAT_ERR_NO_MEMORY; }
}

int pat_tree_build_ragged(pat_tree* t, const int32_t* seq_lens, const int32_t* flat_pages,
                          const int64_t* offsets, int num_seqs) {
    if (!t) return PAT_ERR_BAD_ARGUMENT;
    try {
        return t->tree.build_ragged(seq_lens, flat_pages, offsets, num_seqs);
    } catch (...) { return PAT_ERR_NO_MEMORY; }
}

int pat_tree_pack(pat_tree* t, const int32_t* mnws, int num_mnws, int hratio, int kv_heads,
                  int use_compute_model) {
    if (!t) return PAT_ERR_BAD_ARGUMENT;
    try {
        return t->tree.pack(mnws, num_mnws, hratio, kv_heads, use_compute_model != 0);
    } catch (...) { return PAT_ERR_NO_MEMORY; }
}

int pat_tree_num_buckets(const pat_tree* t) { return t ? static_cast<int>(t->tree.buckets().size()) : 0; }

int pat_tree_bucket(const pat_tree* t, int index, pat_bucket_view* out) {
    if (!t || !out || index < 0 || index >= static_cast<int>(t->tree.buckets().size())) return PAT_ERR_BAD_ARGUMENT;
    const pat::Bucket& b = t->tree.buckets()[index];
    out->mnw[0] = b.mnw[0]; out->mnw[1] = b.mnw[1]; out->mnw[2] = b.mnw[2];
    out->ctas = b.ctas; out->max_seqs = b.max_seqs; out->max_blocks = b.max_blocks;
    out->q_table = b.q_table.data(); out->block_table = b.block_table.data();
    out->num_seqs = b.num_seqs.data(); out->cta_ranks = b.ranks.data(); out->kv_in_cta = b.kv_lens.data();
    return PAT_OK;
}

const int32_t* pat_tree_split_per_seq(const pat_tree* t, int* batch) {
    if (!t) return nullptr;
    if (batch) *batch = static_cast<int>(t->tree.split_per_seq().size());
    return t->tree.split_per_seq().data();
}

int pat_tree_maxima(const pat_tree* t, int32_t out[3]) {
    if (!t || !out) return PAT_ERR_BAD_ARGUMENT;
    out[0] = t->tree.max_split_per_seq();
    out[1] = t->tree.max_seqs_in_cta();
    out[2] = t->tree.max_blocks_in_cta();
    return PAT_OK;
}

int pat_tree_num_nodes(const pat_tree* t) { return t ? static_cast<int>(t->tree.nodes().size()) : 0; }

int pat_tree_node(const pat_tree* t, int node, int32_t out[4]) {
    if (!t || !out || node < 0 || node >= static_cast<int>(t->tree.nodes().size())) return PAT_ERR_BAD_ARGUMENT;
    const pat::TreeNode& n = t->tree.nodes()[node];
    out[0] = n.parent; out[1] = n.s_value; out[2] = n.length;
    if (t->tree.semantics() == pat::Semantics::kPython) out[3] = n.num_pages;
    else out[3] = n.pages ? (n.length + t->tree.block_size() - 1) / t->tree.block_size() : 0;
    return PAT_OK;
}

int pat_tree_node_seqs(const pat_tree* t, int node, const int32_t** seqs, int* count) {
    if (!t || !seqs || !count || node < 0 || node >= static_cast<int>(t->tree.nodes().size())) return PAT_ERR_BAD_ARGUMENT;
    const pat::TreeNode& n = t->tree.nodes()[node];
    *seqs = n.seq_indices.data();
    *count = static_cast<int>(n.seq_indices.size());
    return PAT_OK;
}

int pat_tree_node_pages(const pat_tree* t, int node, const int32_t** pages, int* count) {
    int32_t info[4];
    const int rc = pat_tree_node(t, node, info);
    if (rc != PAT_OK || !pages || !count) return PAT_ERR_BAD_ARGUMENT;
    *pages = t->tree.nodes()[node].pages;
    *count = info[3];
    return PAT_OK;
}

int pat_tree_node_children(const pat_tree* t, int node, int32_t* out, int cap) {
    if (!t || node < 0 || node >= static_cast<int>(t->tree.nodes().size())) return PAT_ERR_BAD_ARGUMENT;
    try {
        const std::vector<int> kids = t->tree.children_in_order(node);
        for (int i = 0; i < static_cast<int>(kids.size()) && i < cap; ++i) out[i] = kids[i];
        return static_cast<int>(kids.size());
    } catch (...) { return PAT_ERR_NO_MEMORY; }
}

pat_work* pat_work_create(const pat_plan_bucket* buckets, int num_buckets, int batch, int hratio,
                          int kv_heads, int page_size, int64_t num_cache_pages,
                          const pat_work_options* options, int* status) {
    int dummy;
    if (!status) status = &dummy;
    pat_work* w = new (std::nothrow) pat_work();
    if (!w) { *status = PAT_ERR_NO_MEMORY; return nullptr; }
    try {
    std::vector<pat::PlanBucketView> views(num_buckets > 0 ? num_buckets : 0);
    for (int i = 0; i < num_buckets; ++i) {
        views[i].ctas = buckets[i].ctas;
        views[i].q_table = buckets[i].q_table;
        views[i].q_stride = buckets[i].q_stride;
        views[i].block_table = buckets[i].block_table;
        views[i].block_stride = buckets[i].block_stride;
        views[i].num_seqs = buckets[i].num_seqs;
        views[i].kv_lens = buckets[i].kv_in_cta;
    }
    const int rc = w->list.build(views.data(), num_buckets, batch, hratio, kv_heads, page_size,
                                 num_cache_pages, to_options(options));
    *status = map_work_error(rc);
    if (rc != 0) { delete w; return nullptr; }
    return w;
    } catch (...) {
        delete w;
        *status = PAT_ERR_NO_MEMORY;
        return nullptr;
    }
}

pat_work* pat_work_from_tree(const pat_tree* t, int hratio, int kv_heads, int64_t num_cache_pages,
                             const pat_work_options* options, int* status) {
    return pat_work_from_tree_multi(t, hratio, kv_heads, 1, num_cache_pages, options, status);
}

pat_work* pat_work_from_tree_multi(const pat_tree* t, int hratio, int kv_heads, int q_per_req,
                                   int64_t num_cache_pages, const pat_work_options* options, int* status) {
    int dummy;
    if (!status) status = &dummy;
    if (!t) { *status = PAT_ERR_BAD_ARGUMENT; return nullptr; }
    pat_work* w = new (std::nothrow) pat_work();
    if (!w) { *status = PAT_ERR_NO_MEMORY; return nullptr; }
    try {
        const int rc = w->list.build_from_tree(t->tree, hratio, kv_heads, num_cache_pages, to_options(options),
                                               q_per_req);
        *status = map_work_error(rc);
        if (rc != 0) { delete w; return nullptr; }
        return w;
    } catch (...) {
        delete w;
        *status = PAT_ERR_NO_MEMORY;
        return nullptr;
    }
}

int pat_tree_advance(pat_tree* t, const int32_t* seq_lens, const int32_t* block_table, int num_seqs,
                     int row_stride) {
    if (!t) return PAT_ERR_BAD_ARGUMENT;
    try {
        std::vector<pat::Growth> growth;
        const int rc = t->tree.plan_advance(seq_lens, block_table, num_seqs, row_stride, growth);
        if (rc != 1) return rc < 0 ? PAT_ERR_BAD_ARGUMENT : 0;
        t->tree.apply_advance(growth);
        return 1;
    } catch (...) { return PAT_ERR_NO_MEMORY; }
}

int pat_work_advance(pat_work* w, pat_tree* t, const int32_t* seq_lens, const int32_t* block_table,
                     int num_seqs, int row_stride) {
    if (!w || !t) return PAT_ERR_BAD_ARGUMENT;
    try {
        std::vector<pat::Growth> growth;
        const int rc = t->tree.plan_advance(seq_lens, block_table, num_seqs, row_stride, growth);
        if (rc != 1) return rc < 0 ? PAT_ERR_BAD_ARGUMENT : 0;
        if (w->list.header().batch != t->tree.batch() || w->list.can_advance(growth) != 1) return 0;
        w->list.advance(growth);        // the page pointers in `growth` point into the caller's table
        t->tree.apply_advance(growth);
        return 1;
    } catch (...) { return PAT_ERR_NO_MEMORY; }
}

void pat_work_destroy(pat_work* w) { delete w; }

int pat_work_get_header(const pat_work* w, pat_work_header* out) {
    if (!w || !out) return PAT_ERR_BAD_ARGUMENT;
    copy_header(w->list.header(), out);
    return PAT_OK;
}

const int32_t* pat_work_blob(const pat_work* w, size_t* words) {
    if (!w) return nullptr;
    if (words) *words = w->list.blob().size();
    return w->list.blob().data();
}

}  // extern "C"

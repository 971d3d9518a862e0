// TEST INFRASTRUCTURE ONLY.  C shim around the reference's own header-only C++
// scheduler (csrc/prefix_tree.h, included from the read-only reference checkout at
// build time; no reference source is copied).  Built by oracle/build_ref.py into
// oracle/_ref/libpat_ref_tree.so and used to freeze golden plans of the C++
// semantics and to cross-check the native scheduler when the checkout is present.
#include <map>
#include <memory>
#include <optional>

#include <torch/torch.h>

#include "prefix_tree.h"

extern "C" {

void* ref_tree_create(int block_size) { return new PrefixTree(block_size); }
void ref_tree_destroy(void* t) { delete static_cast<PrefixTree*>(t); }

void ref_tree_build(void* t, const int* seq_lens, const int* table, int num_seqs, int max_blocks) {
    static_cast<PrefixTree*>(t)->build_radix_tree(seq_lens, table, num_seqs, max_blocks);
}

void ref_tree_pack(void* t, const int* mnws, int n_mnw, int hratio, int kvhead) {
    std::optional<std::vector<std::vector<int>>> shapes;
    if (n_mnw > 0) {
        std::vector<std::vector<int>> v;
        for (int i = 0; i < n_mnw; ++i) v.push_back({mnws[3 * i], mnws[3 * i + 1], mnws[3 * i + 2]});
        shapes = v;
    }
    static_cast<PrefixTree*>(t)->pack_schedule(shapes, hratio, kvhead, false);
}

int ref_tree_num_buckets(void* t) { return (int)static_cast<PrefixTree*>(t)->_internal_info.MNWs.size(); }

// out[0..2] = MNW, out[3] = CTAs, out[4] = q width, out[5] = block width
void ref_tree_bucket_shape(void* t, int i, int* out) {
    auto& k = static_cast<PrefixTree*>(t)->_internal_info;
    out[0] = k.MNWs[i][0]; out[1] = k.MNWs[i][1]; out[2] = k.MNWs[i][2];
    out[3] = (int)k.q_tables[i].size(0);
    out[4] = (int)k.q_tables[i].size(1);
    out[5] = (int)k.block_tables[i].size(1);
}
const int* ref_tree_q(void* t, int i) { return static_cast<PrefixTree*>(t)->_internal_info.q_tables[i].data_ptr<int>(); }
const int* ref_tree_blocks(void* t, int i) { return static_cast<PrefixTree*>(t)->_internal_info.block_tables[i].data_ptr<int>(); }
const int* ref_tree_num_seqs(void* t, int i) { return static_cast<PrefixTree*>(t)->_internal_info.num_seqs_per_CTAs[i].data_ptr<int>(); }
const int* ref_tree_ranks(void* t, int i) { return static_cast<PrefixTree*>(t)->_internal_info.CTA_ranks[i].data_ptr<int>(); }
const int* ref_tree_kv(void* t, int i) { return static_cast<PrefixTree*>(t)->_internal_info.kv_in_CTAs[i].data_ptr<int>(); }
const int* ref_tree_split(void* t, int* n) {
    auto* p = static_cast<PrefixTree*>(t);
    *n = (int)p->split_per_seq.size();
    return p->split_per_seq.data();
}
// out[0..2] = max_split_per_seq, max_seqs_in_CTA, max_blocks_in_CTA
void ref_tree_maxima(void* t, int* out) {
    auto& k = static_cast<PrefixTree*>(t)->_internal_info;
    out[0] = k.max_split_per_seq; out[1] = k.max_seqs_in_CTA; out[2] = k.max_blocks_in_CTA;
}
int ref_tree_num_nodes(void* t) { return (int)static_cast<PrefixTree*>(t)->nodes.size(); }
// out[0..2] = parent, s_value, length
void ref_tree_node(void* t, int i, int* out) {
    auto& n = static_cast<PrefixTree*>(t)->nodes[i];
    out[0] = n.parent; out[1] = n.s_value; out[2] = n.length;
}

}  // extern "C"

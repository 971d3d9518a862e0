/* pat_b200 - C ABI of the B200 prefix-aware decode-attention path.
 *
 * Plain C, no torch types: pointers, sizes, strides (in elements) and a CUDA
 * stream handle.  Every function returns 0 on success or a negative pat_status
 * (pat_b200_strerror gives the text); nothing throws, exits or traps.
 *
 * Each entry point names the reference interface it replaces
 * (paths relative to the reference checkout).
 */
#ifndef PAT_B200_H_
#define PAT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum pat_status {
    PAT_OK = 0,
    PAT_ERR_BAD_ARGUMENT = -1,
    PAT_ERR_EMPTY_QUERY_BOX = -2,    /* Python semantics: IndexError in the reference */
    PAT_ERR_ZERO_QUERIES_PER_BOX = -3, /* Python semantics: max M < HRatio */
    PAT_ERR_UNKNOWN_BUCKET = -4,     /* Python semantics: KeyError in the reference */
    PAT_ERR_NOT_BUILT = -5,
    PAT_ERR_BAD_PLAN = -10,          /* plan tables inconsistent (index out of range ...) */
    PAT_ERR_UNSUPPORTED = -11,       /* dtype / head_dim / head ratio / alignment not supported */
    PAT_ERR_WORKSPACE = -12,         /* workspace missing, too small or not 32-byte aligned */
    PAT_ERR_CUDA = -13,              /* a CUDA runtime or driver call failed */
    PAT_ERR_NO_DEVICE_CODE = -14,    /* the GPU is not an sm_100 part */
    PAT_ERR_TOO_LARGE = -15,         /* size beyond a fixed limit */
    PAT_ERR_NO_MEMORY = -16          /* host allocation failed (no C++ exception leaves the library) */
} pat_status;

const char* pat_b200_strerror(int status);
/* Library version, bumped on any ABI change. */
int pat_b200_abi_version(void);

/* ------------------------------------------------------------------------- *
 * Scheduler: radix tree over physical page ids + tile-plan packer (host).
 * Replaces class PrefixTree of csrc/prefix_tree.h:63-324 as bound by
 * csrc/bindings.cpp:100-146 (PrefixTreeCPP), and can also reproduce
 * prefix_attn/prefix_tree.py:47-616 bit for bit.
 * ------------------------------------------------------------------------- */
typedef struct pat_tree pat_tree;

enum { PAT_SEMANTICS_PYTHON = 0, PAT_SEMANTICS_CPP = 1 };

/* csrc/bindings.cpp:101  PrefixTreeCPP(block_size) */
pat_tree* pat_tree_create(int block_size, int semantics);
void pat_tree_destroy(pat_tree* t);

/* csrc/bindings.cpp:103-126 / csrc/prefix_tree.h:84-101  build_radix_tree(seq_lens, block_table):
 * padded int32 table [num_seqs, row_stride]; row i is cut to ceil(seq_lens[i]/block_size) pages.
 * The table is copied; the caller may free it as soon as the call returns. */
int pat_tree_build(pat_tree* t, const int32_t* seq_lens, const int32_t* block_table,
                   int num_seqs, int row_stride);
/* prefix_attn/prefix_tree.py:146-149  build_radix_tree(seq_lens, list of unpadded lists):
 * row i is flat_pages[offsets[i] .. offsets[i+1]). */
int pat_tree_build_ragged(pat_tree* t, const int32_t* seq_lens, const int32_t* flat_pages,
                          const int64_t* offsets, int num_seqs);

/* csrc/bindings.cpp:128-144 / csrc/prefix_tree.h:183-324 / prefix_tree.py:548-616
 * pack_schedule(MNWs, HRatio, kvHead, use_compute_model).  mnws = num_mnws x 3 ints or NULL/0
 * for the 11 default tile shapes. */
int pat_tree_pack(pat_tree* t, const int32_t* mnws, int num_mnws, int hratio, int kv_heads,
                  int use_compute_model);

/* Plan accessors (struct KernelInfo, csrc/prefix_tree.h:7-25).  Pointers stay valid until the
 * next pack / destroy. */
typedef struct pat_bucket_view {
    int32_t mnw[3];
    int32_t ctas;
    int32_t max_seqs;            /* row width of q_table */
    int32_t max_blocks;          /* row width of block_table */
    const int32_t* q_table;      /* [ctas, max_seqs]  zero padded */
    const int32_t* block_table;  /* [ctas, max_blocks] zero padded */
    const int32_t* num_seqs;     /* [ctas] */
    const int32_t* cta_ranks;    /* [ctas] */
    const int32_t* kv_in_cta;    /* [ctas] */
} pat_bucket_view;

int pat_tree_num_buckets(const pat_tree* t);
int pat_tree_bucket(const pat_tree* t, int index, pat_bucket_view* out);
/* num_split_per_seq [batch]; *batch receives the length */
const int32_t* pat_tree_split_per_seq(const pat_tree* t, int* batch);
/* out[0..2] = max_split_per_seq, max_seqs_in_CTA, max_blocks_in_CTA */
int pat_tree_maxima(const pat_tree* t, int32_t out[3]);

/* Tree inspection (the Python class exposes the same arrays, prefix_tree.py:50-58). */
int pat_tree_num_nodes(const pat_tree* t);
/* out[0..3] = parent, s_value, length, number of pages on the edge */
int pat_tree_node(const pat_tree* t, int node, int32_t out[4]);
int pat_tree_node_seqs(const pat_tree* t, int node, const int32_t** seqs, int* count);
int pat_tree_node_pages(const pat_tree* t, int node, const int32_t** pages, int* count);
/* children in the order the packer visits them; returns the count (<= cap are written) */
int pat_tree_node_children(const pat_tree* t, int node, int32_t* out, int cap);

/* ------------------------------------------------------------------------- *
 * Work list: reference-format plan -> device work items (host).
 * No counterpart as a function in the reference: there a box IS the CTA
 * (csrc/pat_fwd_launch_template.h:35-50, csrc/block_info.h:14-39).
 * ------------------------------------------------------------------------- */
typedef struct pat_work pat_work;

typedef struct pat_plan_bucket {
    int32_t ctas;
    int32_t q_stride;
    int32_t block_stride;
    int32_t reserved;
    const int32_t* q_table;
    const int32_t* block_table;
    const int32_t* num_seqs;
    const int32_t* kv_in_cta;
} pat_plan_bucket;

typedef struct pat_work_options {
    int32_t num_sms;             /* 0 = 148 */
    int32_t dense_min_rows;      /* segments with >= this many query rows use the dense kernel; 0 = default */
    int32_t chunk_tokens_min;    /* 0 = default */
    int32_t chunk_tokens_max;    /* 0 = default */
    int32_t dense_piece_tokens_min; /* a dense CTA share is not cut below about this; 0 = default */
    int32_t items_per_sm;        /* 0 = default */
    int32_t disable_dense;       /* 1 = every segment goes through the streaming kernel */
    int32_t dense_tile_ns;       /* estimated time of one 128-token dense tile; sizes the dense kernel's share
                                    of the SMs when it runs beside the streaming kernel.  0 = default,
                                    < 0 = the dense kernel gets every SM */
    int32_t grow_slack_pages;    /* lists built from a tree: free page slots kept behind the page list of
                                    every request's own last segment, so that pat_work_advance can append
                                    pages in place.  0 = default (8), < 0 = none */
    int32_t reserved;
} pat_work_options;

typedef struct pat_work_header {
    int32_t batch, hratio, page_size, kv_heads;
    int32_t num_stream_items;       /* streaming items (<= 16 query rows, run for every KV head) */
    int32_t num_dense_items;        /* dense items (<= 256 rows, one KV head each), grouped by CTA */
    int32_t num_dense_ctas;         /* persistent CTAs of the dense kernel */
    int32_t num_entries;            /* partial slots; one slot = hratio rows of (head_dim + 1) floats */
    int32_t max_entries_per_list;
    int32_t items_off, queries_off, pages_off, dense_cta_off, merge_indptr_off, merge_entries_off;
    int32_t blob_words, num_segments, max_page_id;
    int64_t unique_tokens;          /* valid tokens summed over segments: every page counted once */
    int64_t stream_tokens;          /* tokens read by streaming items (a segment counts once per row chunk) */
    int64_t dense_tokens;           /* same for dense items */
    int64_t stream_unique_tokens;   /* unique tokens of the segments the streaming kernel handles */
    int64_t dense_unique_tokens;
    int32_t q_per_req;              /* query tokens per request the list was built for (1 = decode) */
    int32_t limits_off;             /* per-(segment, query) visible-token limits, or -1 */
    int32_t dense_q_off;            /* query ids of the dense items, dense_q_width per item, -1 padded */
    int32_t dense_q_width;
} pat_work_header;

/* Returns NULL and sets *status on failure. num_cache_pages > 0 enables a range check of page ids. */
pat_work* pat_work_create(const pat_plan_bucket* buckets, int num_buckets, int batch, int hratio,
                          int kv_heads, int page_size, int64_t num_cache_pages,
                          const pat_work_options* options, int* status);
/* Straight from a built tree (pat_tree_build; packing is not needed): every edge of the radix
 * tree is one segment - its pages, attended by the requests that pass through it. */
pat_work* pat_work_from_tree(const pat_tree* t, int hratio, int kv_heads, int64_t num_cache_pages,
                             const pat_work_options* options, int* status);
/* Several query tokens per request (speculative decoding, a short chunk of prefill on top of a
 * cached prefix; the reference sends such steps to vLLM's flash-attention instead and asserts
 * max_decode_query_len <= 1, plugin/vllm/attention/backends/prefix_attn.py:877-904).  The tree is
 * built from the requests' FULL lengths, the q_per_req new tokens included and already in the
 * cache; position t of a request of length L attends to its first L - q_per_req + 1 + t tokens.
 * In the resulting list a query is a (request, position) pair, id = request * q_per_req + position,
 * and header.batch counts pairs.  Such a list cannot be advanced in place. */
pat_work* pat_work_from_tree_multi(const pat_tree* t, int hratio, int kv_heads, int q_per_req,
                                   int64_t num_cache_pages, const pat_work_options* options, int* status);
/* One decode step later: the same requests, each with seq_lens[i] >= before and its table row
 * extended by the pages the new tokens need (the reference rebuilds tree, plan and tables from
 * scratch every step: prefix_attn/async_tree.py:23-30, and leaves them stale on multi-step
 * decode: plugin/vllm/attention/backends/prefix_attn.py:430-438).  When every request that grew
 * ends in a tree leaf of its own and the new pages fit the slack of the work list, tree and work
 * list (blob and header: fetch them again) are updated in place and the call returns 1; the
 * tree then equals the tree a fresh pat_tree_build of the new tables produces (its packed plan is
 * dropped: pack again to get it).  Returns 0, with nothing changed, when the batch has to be
 * rebuilt (other requests, a changed row, a shared last segment, slack used up); < 0 on a bad
 * argument.  pat_tree_advance does the same for a tree alone. */
int pat_work_advance(pat_work* w, pat_tree* t, const int32_t* seq_lens, const int32_t* block_table,
                     int num_seqs, int row_stride);
int pat_tree_advance(pat_tree* t, const int32_t* seq_lens, const int32_t* block_table, int num_seqs,
                     int row_stride);
void pat_work_destroy(pat_work* w);
int pat_work_get_header(const pat_work* w, pat_work_header* out);
/* int32 blob to copy to the device as is; *words receives its length */
const int32_t* pat_work_blob(const pat_work* w, size_t* words);

/* ------------------------------------------------------------------------- *
 * Decode attention on the device.
 * Replaces pat::pat_mha_fwd_kvcache (csrc/api.h:110-295) and the launcher
 * pat_run_mha_fwd_splitkv_dispatch (csrc/pat_fwd_launch_template.h:52-98).
 * ------------------------------------------------------------------------- */
enum { PAT_DTYPE_FP16 = 0, PAT_DTYPE_BF16 = 1 };
enum { PAT_SKIP_STREAM = 1, PAT_SKIP_DENSE = 2, PAT_SKIP_MERGE = 4,
       PAT_NO_OVERLAP = 16     /* do not let the streaming kernel start while the dense kernel runs */ };

typedef struct pat_decode_args {
    /* tensors (device pointers), strides in elements, last dimension contiguous */
    const void* q;        /* [batch, 1, num_q_heads, head_dim] */
    const void* k_cache;  /* [num_pages, page_size, num_kv_heads, head_dim] */
    const void* v_cache;
    void* out;            /* [batch, 1, num_q_heads, head_dim], same dtype as q */
    float* lse_out;       /* optional [batch, num_q_heads]: natural-log LSE of the scaled scores */
    int64_t q_batch_stride, q_head_stride;   /* (query tokens per request > 1: see q_pos_stride below) */
    int64_t k_page_stride, k_row_stride, k_head_stride;
    int64_t v_page_stride, v_row_stride, v_head_stride;
    int64_t out_batch_stride, out_head_stride;
    int32_t batch, num_q_heads, num_kv_heads, head_dim;
    int32_t page_size;
    int32_t dtype;        /* PAT_DTYPE_* */
    int64_t num_pages;
    float softmax_scale;
    int32_t flags;        /* diagnostics: PAT_SKIP_* bits leave phases out (the result is then
                             incomplete; used to time one kernel at a time) */
    /* work list */
    const int32_t* work_blob;   /* device copy of pat_work_blob */
    pat_work_header work;       /* host copy of the header */
    /* Scratch of pat_b200_workspace_bytes(...) bytes, 32-byte aligned: 256 bytes of control words,
     * then the per-(item, query, KV head) partial results.  The control words must be zero when a
     * workspace is used for the first time; every call that completes leaves them zero again (clear
     * them after a call that reported a failed wait).  Calls that may overlap on the GPU need
     * workspaces of their own. */
    void* workspace;
    size_t workspace_bytes;
    /* Optional device int32[4].  It must hold zeros when the call starts (the library does not
     * clear it: a non-zero word makes the dense kernel's CTAs return at once, as they do after a
     * failure inside the same call).  [0] != 0 after the call means that a bounded wait inside a
     * kernel gave up and `out` is not valid. */
    int32_t* status_word;
    /* limit of every wait inside the kernels, in microseconds; 0 = one second */
    int32_t wait_limit_us;
    /* Query tokens per request; 0 or 1 = decode.  With T > 1, q and out are
     * [batch, T, num_q_heads, head_dim] with the position strides below, `batch` is the number of
     * requests, lse_out is [batch, T, num_q_heads], and the work list must come from
     * pat_work_from_tree_multi with the same T. */
    int32_t q_per_req;
    int64_t q_pos_stride, out_pos_stride;
} pat_decode_args;

size_t pat_b200_workspace_bytes(const pat_work_header* work, int num_q_heads, int head_dim);
/* Enqueues the kernels on `stream` (a cudaStream_t) of the current device and returns. */
int pat_b200_decode(const pat_decode_args* args, void* stream);
/* Number of kernels the last successful pat_b200_decode call on this thread launched. */
int pat_b200_last_launch_count(void);

/* Decode for callers that cannot allocate device memory - a serving engine that has handed the
 * whole GPU to its own memory pool, or a decode loop where a device allocation could block,
 * synchronise or fail.  (It has no counterpart in the reference, which allocates its partial
 * buffers inside every call, csrc/api.h:217-238.)
 *
 * Same arguments and result as pat_b200_decode, except that args->workspace and
 * args->workspace_bytes are ignored: the per-(item, query) partial results go to a fixed array
 * of PAT_B200_STATIC_SCRATCH_BYTES that is part of the library's device image (each GPU that
 * loads the library holds that much memory until the process exits).  A work list that needs
 * more (pat_b200_workspace_bytes(...) > PAT_B200_STATIC_SCRATCH_BYTES) is refused with
 * PAT_ERR_TOO_LARGE and nothing is launched.  The call itself allocates nothing.
 *
 * The first call on each device looks up the array's device address (with that device current);
 * make that first call outside of any stream capture.
 * All calls on a device share the one array and it keeps whatever the previous call left there.
 * Nothing in it has to start at zero - every slot the merge reads is written earlier in the same
 * call - but two calls whose kernels overlap on the GPU (different streams, or different host
 * threads) would overwrite each other's partial results: run them one after the other. */
#define PAT_B200_STATIC_SCRATCH_BYTES (32u << 20)
int pat_b200_decode_static_scratch(const pat_decode_args* args, void* stream);

/* Self-test of the kernels' bounded waits (no counterpart in the reference, whose kernels wait
 * without a limit): launches one thread that waits on a barrier nobody arrives on, with nothing
 * asynchronous in flight.  After the stream has drained, status_word[0] == 99 says that the wait
 * gave up and the kernel returned, status_word[1] holds the nanoseconds it waited.
 * limit_us in (0, 1 000 000]. */
int pat_b200_selftest_wait(int32_t limit_us, int32_t* status_word, void* stream);

/* ------------------------------------------------------------------------- *
 * KV-cache append: the step right before decode attention.
 * Replaces vLLM's reshape_and_cache_flash as called from the reference's serving backend
 * (plugin/vllm/attention/backends/prefix_attn.py:828-837): the K and V rows of the new tokens
 * are written into the paged caches at slot_mapping[token] = page * page_size + row.  A
 * negative slot (vLLM's padding id) is skipped, and so is a slot beyond the cache.
 * 16-bit caches only (kv_cache_dtype "auto"); rows are copied bit for bit.
 * ------------------------------------------------------------------------- */
typedef struct pat_append_args {
    const void* key;               /* [num_tokens, num_kv_heads, head_dim] */
    const void* value;
    void* k_cache;                 /* [num_pages, page_size, num_kv_heads, head_dim] */
    void* v_cache;
    const int64_t* slot_mapping;   /* device, [num_tokens] */
    /* strides in elements (multiples of 8), last dimension contiguous, 16-byte aligned bases */
    int64_t key_token_stride, key_head_stride, value_token_stride, value_head_stride;
    int64_t k_page_stride, k_row_stride, k_head_stride;
    int64_t v_page_stride, v_row_stride, v_head_stride;
    int64_t num_pages;
    int32_t num_tokens, num_kv_heads, head_dim, page_size;
    int32_t dtype;                 /* PAT_DTYPE_* */
    int32_t reserved;
} pat_append_args;

int pat_b200_append_kv(const pat_append_args* args, void* stream);

/* ------------------------------------------------------------------------- *
 * KV-head sharding: head order after the optional all-gather of the outputs.
 * The reference has no multi-GPU path of its own (a tensor-parallel vLLM hands its backend
 * per-rank head counts, plugin/vllm/attention/backends/prefix_attn.py:617-618, and never gathers).
 * staged: what an all-gather of the ranks' [batch, 1, heads_per_rank, head_dim] outputs returns,
 * [world][batch][heads_per_rank][head_dim]; full: [batch][1][world * heads_per_rank][head_dim],
 * heads in rank order.  16-bit elements, 16-byte aligned buffers.
 * ------------------------------------------------------------------------- */
int pat_b200_reorder_heads(const void* staged, void* full, int world, int batch, int heads_per_rank,
                           int head_dim, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PAT_B200_H_ */

// C ABI of libferrule_b200.so.  Every entry point is `extern "C"`, takes plain
// pointers / integers plus the CUDA stream as `void*`, launches asynchronously on
// that stream and returns an FB_* code.  Python binds these through ctypes
// (ferrule_b200/ops/_lib.py); argument structs are mirrored there field for field.
//
// Plays the role of the reference's same-checkout POD ABI between its device runtime
// and native kernels (crates/ferrule-backend/native/cuda/abi/core_provider.h:477-557,
// cutlass_provider.h:390-456).
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  FB_OK = 0,
  FB_ERR_SHAPE = 1,   // launcher rejected the arguments (nothing was launched)
  FB_ERR_ALIGN = 2,   // pointer or stride not 16-byte aligned for TMA
  FB_ERR_DRIVER = 3,  // driver entry point missing or tensor-map encode failed
  FB_ERR_LAUNCH = 4,  // cudaLaunch / attribute error
  FB_ERR_RUNTIME = 5, // other CUDA runtime error
  FB_ERR_LIMIT = 6,   // size beyond a fixed capacity
};

// ---- status word -----------------------------------------------------------------
// 16 bytes: {code, where, detail0, detail1}.  code 0 = ok.
int fb_status_bytes(void);

// ---- tcgen05 GEMM ------------------------------------------------------------------
typedef struct FbGemmArgs {
  const void* w;            // bf16 [groups, w_rows_per_group, k] (row pitch ldw elements)
  const void* x;            // bf16 [x_rows, k] (row pitch ldx elements)
  void* out;
  long long ldw;
  long long w_group_stride; // elements between groups
  long long ldx;
  long long ldo;
  int n_out;                // output channels per group
  int k;
  int groups;
  int w_rows_per_group;
  int x_rows;
  int ntok;                 // rows per tile: 16, 32, 64, 128 or 256
  int epilogue;             // 0 store, 1 swiglu (dual weights), 2 scatter, 3 all-reduce
  int dual_offset;          // row of the "up" block inside a group (epilogue 1)
  int out_fp32;
  int max_tok_tiles;        // capacity of the tile table (grouped mode)
  int x_group_koff;         // batched mode (groups > 1, no tile table): X column offset per group
  int out_group_coff;       // batched mode: output column offset per group
  int force_split;          // 0 = choose automatically; else split-K factor (1, 2, 4, 8)
  const int* tile_group;    // grouped mode: per row-tile expert id, first row, row count
  const int* tile_row0;
  const int* tile_rows;
  const int* num_tok_tiles; // device scalar
  const int* dst_row;       // epilogue 2
  const float* row_scale;   // epilogue 2
  float act_limit;          // epilogue 1: clamp (0 = off)
  int rank;                 // epilogue 3
  int world;
  int rows_cap;
  int flag_capacity;
  void* peer_recv[8];
  void* peer_flags[8];
  void* local_ctr;
  const void* residual;
  long long ldr;
  unsigned long long peer_wait_ns;
  void* status;
  void* trace;              // optional: 8 x uint64 globaltimer stamps written by CTA 0 (profiling)
  int ar_payload_bf16;      // epilogue 3: push partials as bf16 pairs (half the NVLink bytes) instead of fp32
  const int* remap_rank;    // epilogue 2, expert-parallel combine: output row -> destination rank and row of
  const int* remap_row;     //   that rank's bf16 combine buffer (peer_recv[rank], pitch ldo); peer_flags[r][rank]
                            //   is bumped once per call when all of this rank's rows are stored
  void* mc_recv;            // epilogue 3, optional: multicast (NVLS) address of the ranks' receive buffers; partials
                            //   are then broadcast with one multimem store instead of one store per peer
} FbGemmArgs;

int fb_gemm_bf16(const FbGemmArgs* args, void* stream);

// ---- block-scaled FP8 GEMM ---------------------------------------------------------------
typedef struct FbGemmFp8Args {
  const void* w;            // e4m3 [groups, w_rows_per_group, k]
  const void* x;            // e4m3 [x_rows, k]
  const void* w_scale;      // UE8M0 [groups, ceil(w_rows_per_group/128), ceil(k/128)]
  const void* x_scale;      // UE8M0 [x_rows, ldxs] (one per 1 x 128 block)
  void* out;
  long long ldw;            // bytes = elements
  long long w_group_stride;
  long long ldx;
  long long ldxs;
  long long ldo;
  int n_out;
  int k;
  int groups;
  int w_rows_per_group;
  int x_rows;
  int ntok;                 // 16, 32 or 64 (swiglu: 16 or 32)
  int epilogue;             // 0 store, 1 swiglu, 2 scatter
  int dual_offset;          // multiple of 128
  int out_fp32;
  int max_tok_tiles;
  const int* tile_group;
  const int* tile_row0;
  const int* tile_rows;
  const int* num_tok_tiles;
  const int* dst_row;
  const float* row_scale;
  float act_limit;
  int scale_group32;        // 1: w_scale is UE8M0 [groups, w_rows_per_group, k/32] (MXFP4 values in e4m3 containers)
  void* status;
  const int* slot_cnt;      // static row slots instead of a tile table: group g owns rows [g * slot_rows,
  int slot_rows;            //   (g + 1) * slot_rows), slot_cnt[g] of them filled (slot_rows % ntok == 0)
  void* out_scale;          // non-null: `out` gets e4m3 codes (ldo in bytes) and this UE8M0 [rows, ldos] the scale
  long long ldos;           //   of every 1 x 128 output block (store and swiglu epilogues, n_out % 128 == 0)
} FbGemmFp8Args;

int fb_gemm_fp8(const FbGemmFp8Args* args, void* stream);

// ---- paged latent-KV attention -------------------------------------------------------
typedef struct FbAttnArgs {
  const void* q;            // bf16 [rows, heads, kv_lora + rope_dim]
  const void* kv;           // bf16 [pool_rows, kv_lora + rope_dim] (one layer of the pool)
  void* out;                // bf16 [rows, heads, kv_lora]
  const int* block_table;   // [num_seqs, max_blocks]
  const int* row_seq;       // [rows] sequence of each query row
  const int* row_pos;       // [rows] last kv position the row may see
  const float* sink;        // optional [heads]
  float* part_o;            // split scratch [rows, splits, heads, kv_lora] fp32
  float* part_ml;           // split scratch [rows, splits, heads, 2] fp32
  void* status;
  long long ldq;
  long long ldo;
  long long pool_rows;
  int rows;
  int heads;
  int kv_lora;
  int rope_dim;
  int num_seqs;
  int max_blocks;
  int page_size;
  int group_rows;           // consecutive query rows of one sequence sharing a CTA tile (1,2,4,8,16)
  int splits;
  int split_tokens;         // multiple of 64
  float softmax_scale;
  void* merge_ctr;          // optional: zeroed uint32 [ceil(rows/group_rows) * head blocks]; merges in-kernel
  const int* selection;     // optional [rows, sel_width] explicit pool rows per query row, -1 = masked
  int sel_width;            //   (then block_table / row_seq / row_pos are unused and group_rows must be 1)
  void* trace;              // optional uint64 [32]: globaltimer stamps of CTA (0,0,0) (profiling)
  int decode_only;          // the caller asserts: every sequence has exactly one query row in this launch and its
                            // KV rows below row_pos were written before the running step began (plain decode)
} FbAttnArgs;

int fb_mla_attention(const FbAttnArgs* args, void* stream);

// ---- prefill attention on tcgen05 (128-row tiles of (position, head) pairs of one sequence) ----
typedef struct FbPrefillAttnArgs {
  const void* q;            // bf16 [rows, heads, 576] contiguous (ldq == heads * 576)
  const void* kv;           // bf16 [pool_rows, 576] (one layer of the pool)
  void* out;                // bf16 [rows, heads, 512]
  const int* tiles;         // [n_tiles, 4]: sequence, first query row, query rows (<= 128 / heads, consecutive
                            //   positions of that sequence), position of the first row; 16-byte aligned
  const int* block_table;   // [num_seqs, max_blocks]
  const float* sink;        // optional [heads]
  void* status;
  long long ldq;
  long long ldo;
  long long pool_rows;
  int n_tiles;
  int rows;
  int heads;                // must divide 128
  int kv_lora;              // 512
  int rope_dim;             // 64
  int num_seqs;
  int max_blocks;
  int page_size;            // power of two >= 8
  float softmax_scale;
} FbPrefillAttnArgs;

int fb_mla_prefill_tc(const FbPrefillAttnArgs* args, void* stream);

// ---- small fused operators ------------------------------------------------------------
int fb_embedding(const int* ids, const void* table, void* out, int rows, int dim, int vocab,
                 void* status, void* stream);
int fb_add_rmsnorm(const void* x, long long ldx, const void* delta, long long ldd,
                   const void* weight, void* res_out, long long ldr, void* norm_out, long long ldn,
                   int rows, int dim, float eps, void* stream);
// the same, and the normalised rows once more as e4m3 codes q_out [rows, dim] + UE8M0 q_scale [rows, dim / q_block],
// q_block 128 (bit-equal to fb_quant_fp8_rows of norm_out) or 32 (fb_quant_mxfp8_rows); dim % 128 == 0
int fb_add_rmsnorm_q(const void* x, long long ldx, const void* delta, long long ldd,
                     const void* weight, void* res_out, long long ldr, void* norm_out, long long ldn,
                     int rows, int dim, float eps, void* q_out, long long ldq, void* q_scale, long long lds,
                     int q_block, void* stream);
int fb_mla_prep(const void* q, long long ldq, int q_head_dim, const void* ckv, long long ldckv,
                int heads, int kv_lora, int rope_dim, const void* kv_norm_w, float eps,
                const float* cos_t,
                const float* sin_t, int max_pos, const int* positions, const long long* write_slot,
                void* kv_pool, long long pool_rows, void* q_out, long long ldq_out, int rows,
                void* status, void* stream);
int fb_router_topk(const float* logits, long long ldl, const float* bias,
                   const long long* hash_table, const int* token_ids, int rows, int experts,
                   int topk, int score_fn, int n_groups, int topk_groups, int normalize,
                   float route_scale, int* out_idx, float* out_w, void* stream);
int fb_moe_plan(const int* topk_idx, const float* topk_w, int routes, int topk, int e_lo, int e_hi,
                int ntok, int dst_slots, int* src_token, int* dst_row, float* row_scale, int* tile_group,
                int* tile_row0, int* tile_rows, int max_tiles, int* counts, int* meta, void* status,
                void* stream);
// second tile table (another tile height) over the expert-major rows of a plan whose counts are on the device
int fb_moe_retile(const int* counts, int local_experts, int ntok, int* tile_group, int* tile_row0, int* tile_rows,
                  int max_tiles, int* meta, void* status, void* stream);
int fb_router_plan_fused(const void* x, long long ldx, const void* w, int hidden, const float* bias,
                         const long long* hash_table, const int* token_ids, int rows, int experts,
                         int topk, int score_fn, int n_groups, int topk_groups, int normalize,
                         float route_scale, int* out_idx, float* out_w, int e_lo, int e_hi, int ntok,
                         int dst_slots, int* src_token, int* dst_row, float* row_scale, int* tile_group,
                         int* tile_row0, int* tile_rows, int max_tiles, int* counts, int* meta,
                         void* done_ctr, void* status, void* stream);
// asynchronous L2 prefetch of [ptr, ptr + bytes) (ptr 16-byte aligned)
int fb_l2_prefetch(const void* ptr, long long bytes, void* stream);
// decode-sized batches, static plan: expert e (local) owns rows [e * slot_rows, (e + 1) * slot_rows) of src_token /
// dst_row / row_scale / xg; cnt[e] (zeroed by the caller before the step) ends up as its row count
int fb_router_append(const void* x, long long ldx, const void* w, int hidden, const float* bias,
                     const long long* hash_table, const int* token_ids, int rows, int experts, int topk, int score_fn,
                     int n_groups, int topk_groups, int normalize, float route_scale, int* out_idx, float* out_w,
                     int e_lo, int e_hi, int slot_rows, int dst_slots, int* cnt, int* src_token, int* dst_row,
                     float* row_scale, void* xg, long long ldxg, void* status, void* stream);
// the same with a prologue: row = bf16(x + delta) (delta may be null) -> res_out, RMSNorm(row) * norm_w -> norm_out
// and into the router, bit-equal to fb_add_rmsnorm followed by fb_router_append (norm_w null: no prologue)
int fb_norm_router_append(const void* x, long long ldx, const void* delta, long long ldd, const void* norm_w,
                          void* res_out, long long ldr, void* norm_out, long long ldn, float eps, const void* w,
                          int hidden, const float* bias, const long long* hash_table, const int* token_ids, int rows,
                          int experts, int topk, int score_fn, int n_groups, int topk_groups, int normalize,
                          float route_scale, int* out_idx, float* out_w, int e_lo, int e_hi, int slot_rows,
                          int dst_slots, int* cnt, int* src_token, int* dst_row, float* row_scale, void* xg,
                          long long ldxg, void* status, void* stream);
int fb_gather_rows(const void* x, long long ldx, const int* src_token, const int* meta, void* out,
                   long long ldo, int cap_rows, int dim, int src_rows, void* status, void* stream);
int fb_moe_reduce_norm(const void* route_out, int slots, int topk, const int* topk_idx, int e_lo, int e_hi,
                       const void* residual, long long ldr, void* out, long long ldo, int rows, int dim,
                       const void* norm_w, void* norm_out, long long ldn, float eps, void* stream);
int fb_moe_reduce(const void* route_out, int slots, int topk, const int* topk_idx, int e_lo,
                  int e_hi, const void* extra, long long lde, const void* residual, long long ldr,
                  void* out, long long ldo, int out_fp32, int rows, int dim, void* stream);
int fb_argmax(const float* logits, long long ldl, int rows, int vocab, int* out_id, float* out_val,
              void* stream);
int fb_argmax_chunked(const float* logits, long long ldl, int rows, int vocab, int chunks,
                      float* part_val, int* part_id, void* row_ctr, int* out_id, float* out_val,
                      void* stream);
int fb_topk_logits(const float* logits, long long ldl, int rows, int vocab, int k, int* out_id,
                   float* out_val, void* stream);
int fb_copy_pages(void* pool, long long layer_stride, long long page_elems, const int* pairs,
                  int n_pairs, int n_pages, int layers, void* status, void* stream);
// greedy-token feedback between decode steps that run back to back on the device: token_ids[r] = next_id[r]
// (ids outside [0, vocab) become 0); with `advance` the row also moves to the next position and looks its KV
// write slot up in the page list (block_table [num_seqs, max_blocks])
int fb_decode_advance(const int* next_id, int* token_ids, int* positions, int* row_pos, long long* write_slot,
                      const int* row_seq, const int* block_table, int max_blocks, int page_size, int num_seqs,
                      int rows, int vocab, int advance, void* stream);

// fb_norm_router_append that gathers quantised rows: with q_src set, every route's reserved row receives the token's
// codes (q_src [rows, hidden] -> xg_q) and scale bytes (s_src [rows, s_cols] -> xg_s) instead of a bf16 row
int fb_router_append_q(const void* x, long long ldx, const void* delta, long long ldd, const void* norm_w,
                       void* res_out, long long ldr, void* norm_out, long long ldn, float eps, const void* w,
                       int hidden, const float* bias, const long long* hash_table, const int* token_ids, int rows,
                       int experts, int topk, int score_fn, int n_groups, int topk_groups, int normalize,
                       float route_scale, int* out_idx, float* out_w, int e_lo, int e_hi, int slot_rows,
                       int dst_slots, int* cnt, int* src_token, int* dst_row, float* row_scale, void* xg,
                       long long ldxg, const void* q_src, long long ldq, const void* s_src, long long lds, void* xg_q,
                       long long ldxgq, void* xg_s, long long ldxgs, int s_cols, void* status, void* stream);

// ---- collectives through the NVLink switch (multimem) ------------------------------------------------
// mode 1 reduce-scatter (out = this rank's slice [ceil(rows/world), dim]), 2 all-gather (src = this rank's slice),
// 3 all-reduce.  src: route rows [rows * slots, dim] (summed per token as in fb_moe_reduce; slots = 1, topk = 0: a
// plain partial), or null when the partial already sits in the staging area of the current call parity.
// local_base / mc_base: this rank's mapping and the multicast mapping of the channel's symmetric buffer
// [flags (256 B) | stage x 2 | result x 2]; priv: 4 private uint32 (zeroed once).
int fb_mm_collective(const void* src, long long lds, int slots, int topk, const int* topk_idx, int e_lo, int e_hi,
                     const void* residual, long long ldr, void* out, long long ldo, int rows, int dim, int mode,
                     const void* norm_w, void* norm_out, long long ldn, float eps, void* local_base, void* mc_base,
                     long long stage_off, long long result_off, long long buf_bytes, void* priv, int rank, int world,
                     unsigned long long wait_ns, void* status, void* stream);

// ---- data movers (index fills, row copies; see data_movers.cu) ----------------------------------------
int fb_mv_fill(int* dst, long long n, int start, int step, void* stream);
int fb_mv_pack_pairs(const int* ids, const float* vals, int* out, int n, void* stream);
// mode 0 window (positions), 1 offset list (idx [rows, ldi]), 2 counts (idx [rows]); base [rows] int64
int fb_mv_index_fill(int* sel, long long lds, int col0, int rows, int width, int mode, const int* positions,
                     const long long* base, const int* idx, long long ldi, void* stream);
// idx null: dst[dst_row0 + r] = src[r]; else dst[dst_row0 + r] = src[idx[r]]; rows of row_bytes (multiple of 16)
int fb_mv_move_rows(void* dst, long long ldd_bytes, long long dst_row0, const void* src, long long lds_bytes,
                    const int* idx, int rows, int src_rows, int row_bytes, void* status, void* stream);
int fb_mv_scatter_add(float* dst, long long ldd, int dst_rows, const float* src, long long lds, const int* idx,
                      int rows, int dim, void* status, void* stream);
int fb_mv_saxpy(float* y, const float* x, float a, long long n, void* stream);
int fb_mv_ring_to_logical(const int* slots, long long lds, int rows, int width, int window, const int* last_position,
                          const int* n_compressed, int* out_index, int* out_plane, long long ldo, void* stream);
int fb_mv_paged_row_scatter(void* pool, long long pool_rows, int row_bytes, const int* block_table, int max_blocks,
                            int num_seqs, int page_size, const int* row_seq, const int* positions, const void* src,
                            long long lds_bytes, int rows, void* status, void* stream);

// ---- quantisation / packing ---------------------------------------------------------------
int fb_quant_fp8_rows(const void* x, long long ldx, void* q, long long ldq, void* scale, long long lds,
                      int rows, int n, int writeback_bf16, void* stream);
int fb_dequant_fp8_block(const void* q, const void* scale, void* out, int rows, int cols, int block,
                         void* stream);
int fb_quant_mxfp4_rows(const void* x, long long ldx, void* packed, void* scale, int rows, int n,
                        void* stream);
int fb_dequant_mxfp4(const void* packed, const void* scale, void* out, int rows, int n, void* stream);
int fb_hadamard_rows(void* x, long long ldx, int rows, int n, void* stream);

// ---- MXFP4 x MXFP8 block-scaled GEMM (routed experts) --------------------------------------------
typedef struct FbGemmMxfp4Args {
  const void* w;            // packed e2m1 [groups, w_rows_per_group, k / 2] (low nibble = even element), 32-byte aligned
  const void* x;            // e4m3 [x_rows, k]
  const void* w_sf;         // weight scales arranged by fb_mxfp4_prepare_sf
  const void* x_scale;      // UE8M0 [x_rows, k / 32]
  void* out;                // bf16 / fp32 [rows, n_out], or e4m3 codes with out_mode 2
  void* out_scale;          // out_mode 2: UE8M0 [rows, n_out / 32]
  long long ldw_bytes;      // bytes between weight rows (k / 2 when dense)
  long long w_group_stride_bytes;
  long long ldx;
  long long ldxs;
  long long ldo;
  long long ldos;
  int n_out;
  int k;                    // multiple of 128
  int groups;
  int w_rows_per_group;
  int x_rows;
  int ntok;                 // 16, 32, 64 (128 without SwiGLU)
  int epilogue;             // 0 store, 1 SwiGLU (w rows = [gate block | up block]), 2 weighted scatter
  int dual_offset;
  int out_mode;             // 0 bf16, 1 fp32, 2 MXFP8 (e4m3 + one UE8M0 scale per 32 channels; store / SwiGLU only)
  int max_tok_tiles;
  const int* tile_group;
  const int* tile_row0;
  const int* tile_rows;
  const int* num_tok_tiles;
  const int* dst_row;
  const float* row_scale;
  float act_limit;
  void* status;
  int w_tiled;              // w is tile-major: [groups][ceil(rows/128)][k/128][128 rows][64 bytes] (rows padded to 128)
  int w_fp8;                // weights are e4m3 bytes [groups, rows, k] (ldw_bytes = bytes per row) instead of packed e2m1;
                            //   w_sf has the same per-32 layout (128 x 128 block scales replicated)
  const int* slot_cnt;      // static row slots instead of a tile table: group g owns rows [g * slot_rows,
  int slot_rows;            //   (g + 1) * slot_rows), slot_cnt[g] of them filled (slot_rows % ntok == 0)
} FbGemmMxfp4Args;
int fb_gemm_mxfp4(const FbGemmMxfp4Args* args, void* stream);
// linear UE8M0 weight scales [groups, rows, k / 32] -> [groups, ceil(rows / 128), k / 128, 512] blocks for the kernel
// (rows beyond the weight are padded with 0x7f); out holds groups * ceil(rows / 128) * (k / 128) * 512 bytes
int fb_mxfp4_prepare_sf(const void* scale, void* out, int groups, int rows, int k, void* stream);
// bf16 [rows, n] -> e4m3 codes [rows, n] + UE8M0 scales [rows, n / 32] (1 x 32 blocks), n a multiple of 128
int fb_quant_mxfp8_rows(const void* x, long long ldx, void* q, long long ldq, void* scale, long long lds, int rows,
                        int n, void* stream);

// ---- DeepSeek-V4 operators ---------------------------------------------------------------
// hyper-connections: state bf16 [tokens, hc, hidden], fn fp32 [nmix, hc * hidden]; coeff fp32 [tokens, nmix]
// = [pre | post | comb]; nmix = hc (head reduction) or 2 hc + hc^2; hc in {2, 4}
int fb_hc_pre(const void* state, const float* fn, const float* scale, const float* base, void* hidden_out,
              int out_fp32, float* coeff, int tokens, int hc, int hidden, int nmix, float eps, float norm_eps,
              int sinkhorn_iters, void* stream);
// same result with the hc * hidden reduction split over `chunks` CTAs per token (part: tokens * chunks * 32 floats,
// ctr: zeroed uint32 [tokens])
int fb_hc_pre_split(const void* state, const float* fn, const float* scale, const float* base, void* hidden_out,
                    int out_fp32, float* coeff, int tokens, int hc, int hidden, int nmix, float eps, float norm_eps,
                    int sinkhorn_iters, int chunks, float* part, void* ctr, void* stream);
int fb_hc_post(const void* hidden_in, const void* residual, const float* coeff, void* out, int tokens, int hc,
               int hidden, void* stream);
// group g pools rows row0 + g * ratio + [0, window); rows outside [0, n_rows) are masked; kv / gate rows have
// pitch ld, ape is contiguous [ratio, cur_col + dim]; rows of the current group read columns [cur_col, cur_col + dim), rows of the previous one [0, dim)
int fb_compressor_pool(const float* kv, const float* gate, long long ld, const float* ape, void* out, long long ldo,
                       int groups, int dim, int ratio, int window, int row0, int n_rows, int cur_col, void* stream);
int fb_rope_rows(void* x, long long ld_row, long long ld_head, int rows, int heads, int off, int rdim,
                 const int* positions, const float* cos_t, const float* sin_t, int max_pos, int inverse,
                 void* status, void* stream);
int fb_indexer_scores(const void* q, const void* plane, long long ldp, const float* head_w, float* scores,
                      long long ld_s, int queries, int heads, int d, int n, void* stream);
// one draft step of the Markov proposal head: id = argmax_t(logits[t] + W2[t] . W1[*prev_token]), ties -> lower id
int fb_markov_step(const float* logits, const void* w1, const void* w2, int vocab, int rank, int chunks,
                   const int* prev_token, float* part_val, int* part_id, void* ctr, int* out_id, float* out_val,
                   void* status, void* stream);
// taps[t][tap_off : +hidden] = bf16(mean over the hc copies of state[t])
int fb_hc_mean_scatter(const void* state, void* taps, long long ld_taps, int tap_off, int tokens, int hc, int hidden,
                       void* stream);
// head reduction over GEMM-produced dots bf16 [queries * heads, n] (pitch ld): same score chain as fb_indexer_scores
int fb_indexer_reduce(const void* dots, long long ld, const float* head_w, float* scores, long long ld_s, int queries,
                      int heads, int n, void* stream);
// n_visible (per query) may be NULL, then n_fixed applies; k <= 512
int fb_indexer_topk(const float* scores, long long ld_s, const int* n_visible, int n_fixed, int k, int* out_idx,
                    long long ldo, int queries, void* stream);

// ---- stable-slot expert table (streamed routed experts) -------------------------------------
// updates: int4 records {slot, expert, generation, evicted expert or -1}, applied in order
int fb_expert_table_apply(int* expert_to_slot, int* slot_expert, int* slot_gen, const void* updates, int n,
                          int n_experts, int n_slots, void* status, void* stream);
// tile_group: expert ids -> arena slots in place; miss[0] counts tiles of absent experts, miss[1..63] lists them
int fb_expert_table_resolve(int* tile_group, int* tile_rows, const int* num_tiles, int max_tiles,
                            const int* expert_to_slot, int n_experts, int* miss, void* stream);

// ---- expert-parallel MoE over peer memory -------------------------------------------------
// Every rank owns one symmetric buffer with the same layout (byte offsets below):
//   recv_x    bf16 [world][cap][hidden]   rows dispatched to this rank, one segment per source
//   recv_meta int4 [world][cap]           {local expert, return row (token * topk + slot), weight bits, 1}
//   recv_cnt  u32  [world]                rows each source sent in the current call
//   comb      bf16 [tcap * topk][hidden]  weighted expert outputs returned to this rank
//   disp_flag / comb_flag / gath_flag  u32 [world]   arrival counters (one per source rank, only grow)
//   gath_out  bf16 [world][tcap][hidden]  all-gathered layer outputs (optional)
typedef struct FbEpArgs {
  void* base[8];
  long long off_recv_x, off_recv_meta, off_recv_cnt, off_comb, off_disp_flag, off_comb_flag, off_gath_flag,
      off_gath_out;
  int rank, world, cap, hidden, topk, experts_local, tcap;
  unsigned long long wait_ns;
  void* status;
} FbEpArgs;
// cnt_local: u32 [world] zeroed once; every ctr: u32 [2] zeroed once, private to its call site
int fb_ep_dispatch(const FbEpArgs* a, const void* x, long long ldx, const int* idx, const float* wts, int tokens,
                   void* cnt_local, void* ctr, void* stream);
int fb_ep_collect(const FbEpArgs* a, void* ctr, int e_lo, int* r_idx, float* r_w, int* remap_rank, int* remap_row,
                  void* stream);
int fb_ep_combine_reduce(const FbEpArgs* a, void* ctr, const void* extra, long long lde, const void* residual,
                         long long ldr, void* out, long long ldo, int tokens, int allgather, int gather_row0, void* stream);
int fb_ep_gather_wait(const FbEpArgs* a, void* ctr, void* stream);

// ---- peer memory and collectives --------------------------------------------------------
int fb_ipc_handle_bytes(void);
int fb_ipc_alloc(void** ptr, long long bytes, void* handle_out);   // zero-filled device buffer + IPC handle
int fb_ipc_open(const void* handle, void** ptr);                   // map a peer rank's buffer
int fb_ipc_close(void* ptr);
int fb_ipc_free(void* ptr);
// ctr: private device words {calls, ctas_done, consumed arrivals per flag ...}
int fb_moe_reduce_allreduce(const void* route_out, int slots, int topk, const int* topk_idx, int e_lo,
                            int e_hi, const void* residual, long long ldr, void* out, long long ldo,
                            int rows, int dim, int rank, int world, int rows_cap,
                            void* const* peer_recv, void* const* peer_flags, void* ctr,
                            int payload_bf16, unsigned long long wait_ns, void* status, void* stream);
// the same with the receive buffers' multicast address (null: plain peer stores)
int fb_moe_reduce_allreduce_mc(const void* route_out, int slots, int topk, const int* topk_idx, int e_lo,
                               int e_hi, const void* residual, long long ldr, void* out, long long ldo,
                               int rows, int dim, int rank, int world, int rows_cap,
                               void* const* peer_recv, void* const* peer_flags, void* ctr,
                               int payload_bf16, unsigned long long wait_ns, void* mc_recv, void* status,
                               void* stream);
int fb_argmax_allgather(int* ids, float* vals, int vocab_lo, int rows, int rank, int world, int rows_cap,
                        void* const* peer_recv, void* const* peer_flags, void* ctr,
                        unsigned long long wait_ns, void* status, void* stream);
// two ranks bounce a counter through each other's memory; out_ns[0] = total ns for `iters` round trips
int fb_peer_pingpong(void* mine, void* theirs, int iters, int initiator, unsigned long long limit_ns, void* out_ns,
                     void* status, void* stream);
int fb_flag_wait_probe(const void* flag, int target, unsigned long long wait_ns, void* status,
                       int* result, void* stream);

#ifdef __cplusplus
}
#endif

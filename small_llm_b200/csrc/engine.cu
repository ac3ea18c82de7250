// Host engine + C ABI (include/sllm.h) of the B200 token loop.
//
// One engine = one GPU, one stream, every device buffer allocated at creation:
//   weights     re-laid-out at load time (repack.cuh)
//   KV pool     [L][pages][2][H][64][hd], pages handed to slots by the host (block table on device)
//   slot state  tokens, lengths, finished flags, seen-id bitmaps, draw cursors
//   pass state  token list (id, slot, position) of the pass in flight + activations
// A "pass" runs the model over a list of new tokens; a prefill pass carries a chunk of prompt
// tokens, a decode pass one token per slot.  The decode iteration (sampler + pass) is replayed
// as a CUDA graph with programmatic dependent launches between its kernels.
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <random>
#include <string>
#include <tuple>
#include <vector>

#include "../../include/sllm.h"
#include "attn_decode.cuh"
#include "attn_prefill.cuh"
#include "attn_prefill_tc.cuh"
#include "attn_stream.cuh"
#include "common.cuh"
#include "decode_fused.cuh"
#include "decode_persist.cuh"
#include "gemm_tc.cuh"
#include "gemv.cuh"
#include "repack.cuh"
#include "sampler.cuh"

using namespace sllm;

namespace {

thread_local std::string g_create_error;

struct ParamSlot {
    std::string name;
    uint64_t dims[2];
    uint32_t ndim;
    int kind;    // 0 embedding, 1 attn_norm, 2 q, 3 k, 4 v, 5 out, 6 ffn_norm, 7 gate, 8 up, 9 down, 10 final_norm
    int layer;
};

struct GraphKey {
    int n_slots; float t, p, pen; uint32_t eos; long long stop; int seeded; int stride; const void* draws; int iters;
    bool operator<(const GraphKey& o) const {
        return std::tie(n_slots, t, p, pen, eos, stop, seeded, stride, draws, iters) <
               std::tie(o.n_slots, o.t, o.p, o.pen, o.eos, o.stop, o.seeded, o.stride, o.draws, o.iters);
    }
};

}  // namespace

struct sllm_engine {
    sllm_model_config cfg{};
    sllm_engine_options opt{};
    ModelDims md{};
    bool f32 = false;
    int dev = 0;
    int sm_count = 148;
    cudaStream_t stream = nullptr;
    std::string err;

    // weights
    std::vector<ParamSlot> params;
    std::vector<LayerW> layers;
    std::vector<void*> allocs;
    void* emb_w = nullptr;        // [V][D] weight dtype (tied head)
    float* emb_f32 = nullptr;     // [V][D] fp32 (gather)
    float* g_final = nullptr;
    float2* rope = nullptr;
    float* staging = nullptr;     // largest parameter, fp32
    size_t staging_elems = 0;
    uint64_t weight_bytes = 0, kv_bytes = 0, scratch_bytes = 0;

    // KV
    void* kv_pool = nullptr;
    long long n_pages = 0;
    int pages_per_seq = 0;
    std::vector<int> free_pages;
    std::vector<std::vector<int>> slot_pages;
    int* d_block_table = nullptr;

    // slots
    SeqState st{};
    int max_batch = 0;
    int n_live = 0;                    // slots 0..n_live-1 are in use
    std::vector<int> h_len_bound;      // upper bound of each slot's token count (host view)
    std::vector<char> slot_released;   // slot holds no sequence: its block table points at the spare page
    int spare_page = 0;                // never handed out: idle slots write their (ignored) K/V there

    // pass buffers
    int pass_cap = 0;                  // tokens per pass (size of the pass buffers)
    int chunk_tokens = 0;              // prompt positions per prefill chunk (<= pass_cap)
    uint32_t* d_tok_id = nullptr; int* d_tok_slot = nullptr; int* d_tok_pos = nullptr;
    uint32_t* d_dec_id = nullptr; int* d_dec_slot = nullptr; int* d_dec_pos = nullptr;   // decode pass (written by the sampler)
    int* d_attn_order = nullptr;       // decode pass: slots by descending length, the attention grid's block order
    std::vector<int> h_attn_order;
    float* x = nullptr; float* q = nullptr; float* att = nullptr; float* hid = nullptr;
    int* d_row_tok = nullptr;
    float* ss_part = nullptr; int ss_parts = 0;    // folded RMSNorm: [pass_cap][ss_parts] partial sums of squares
    int* d_row_target = nullptr; float* d_row_loss = nullptr;    // sllm_eval_loss: targets and losses of one group of logits rows
    PfTile* d_tiles = nullptr;
    float* step_logits = nullptr;      // [max_batch][V]
    float* pass_logits = nullptr;      // [logit_rows_cap][V]
    int logit_rows_cap = 0;
    // tensor-core path (bf16 weights, passes of >= tc_min_tokens tokens)
    __nv_bfloat16* xn16 = nullptr; __nv_bfloat16* att16 = nullptr; __nv_bfloat16* hid16 = nullptr; __nv_bfloat16* head16 = nullptr;
    unsigned int* d_status = nullptr;
    void* encode_tiled = nullptr;                    // cuTensorMapEncodeTiled
    std::vector<CUtensorMap> map_wqkv, map_wo, map_wgu, map_wd;
    CUtensorMap map_head{};
    CUtensorMap map_kv{};                            // the KV pool as [rows][64] bf16 (head_dim 64): K pages by TMA
    bool attn_tc = false;                            // tensor-core prefill attention usable (bf16, head_dim 64)
    int pf_tile_q = kPfQ;                            // queries per prefill tile (128 with the tensor-core kernel)
    std::map<std::pair<const void*, int>, CUtensorMap> map_x;    // (activation buffer, BN) -> map
    int tc_min_tokens = 2;                           // measured: from 2 tokens on the tensor-core pass beats the GEMV family (0.48 vs 0.51 ms at 2 sequences, 0.53 vs 1.40 ms at 8)
    // fused single-token decode path
    float* xb = nullptr; float* attn_parts = nullptr; float* down_parts = nullptr;
    std::vector<void*> wdT;                          // per layer: down weights as [F][D]
    bool use_attn_stream = true;
    int fused_upc = 0, fused_nb = 0;
    bool fused_ok = false;
    // persistent single-token decode kernel (decode_persist.cuh): bf16 weights, models whose per-block weight slices fit shared memory
    bool persist_ok = false;
    int ps_na = 0, ps_smax = 0, ps_ppsmax = 0;
    size_t ps_smem = 0;
    unsigned long long *ps_xa = nullptr, *ps_xb = nullptr, *ps_qkv = nullptr, *ps_ap = nullptr, *ps_hb = nullptr;
    unsigned int* ps_epoch = nullptr;
    unsigned long long* ps_mxb = nullptr;
    bool fold_sampler = true;           // SLLM_NO_FOLD: the sampler's first two kernels stay kernels of their own
    LayerW* d_layers = nullptr;
    // attention scratch
    float* part_o = nullptr; float* part_ml = nullptr; unsigned int* ticket = nullptr;
    int split_tok_cap = 64;
    int tune_tc_split = 0;             // SLLM_TC_SPLIT: tuning aid, forces the split-K cluster size of the projections
    int tune_no_wide_epi = 0;          // SLLM_NO_WIDE_EPI: the projections keep the thread-per-row epilogue (comparison aid, and the path of models whose row counts are not multiples of 4)
    int tune_no_persistent_tc = 0;     // SLLM_NO_PERSISTENT_TC: the wide projections run one tile per block (comparison aid)
    int order_min_waves = 1;           // the attention grid is ordered by length once its blocks exceed this many waves of 4 per SM (SLLM_ORDER_WAVES; measured: 1.06 -> 1.01 ms per iteration at 64 sequences, 1.61 -> 1.52 at 128, 1.99 -> 1.90 at 192 against a threshold of 4 waves)
    int tune_stream_splits = 0;        // SLLM_STREAM_SPLITS: tuning aid, overrides the split count of the streaming kernel
    unsigned long long* samp_mass = nullptr; unsigned int* samp_cnt = nullptr;   // sampler's level-0 histograms
    float* samp_w = nullptr; float* samp_pmax_val = nullptr; int* samp_pmax_idx = nullptr;
    int samp_bps_cap = 128;
    // draws
    double* d_draws = nullptr; size_t draws_cap = 0;
    // host pinned
    int* h_flags = nullptr;
    // prefill chunk lists: two pinned staging buffers, so that the host builds chunk k + 1 while the GPU runs chunk k
    // (a copy from pageable memory would first synchronise the stream)
    unsigned char* h_pf[2] = {nullptr, nullptr};
    cudaEvent_t ev_pf[2] = {nullptr, nullptr};
    bool ev_pf_used[2] = {false, false};
    int pf_next = 0;

    // graphs
    std::map<GraphKey, std::pair<cudaGraphExec_t, int>> graphs;   // exec + kernels per replay

    uint64_t launches = 0, decode_steps = 0, prefill_tokens = 0;
    int iter_launches = 0;             // kernels in the decode-iteration graph captured last
    float last_step_ms = 0.f;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    std::vector<cudaEvent_t> step_events;      // sllm_decode_loop_timed
    size_t max_dyn_smem = 0;
};

namespace {

#define CU(call)                                                                                   \
    do {                                                                                           \
        cudaError_t _e = (call);                                                                   \
        if (_e != cudaSuccess) {                                                                   \
            char _b[512];                                                                          \
            std::snprintf(_b, sizeof _b, "CUDA error %s at %s:%d: %s", cudaGetErrorName(_e), __FILE__, __LINE__, \
                          cudaGetErrorString(_e));                                                 \
            e->err = _b;                                                                           \
            return SLLM_ERR_CUDA;                                                                  \
        }                                                                                          \
    } while (0)

int fail(sllm_engine* e, int code, const std::string& msg) {
    if (e) e->err = msg; else g_create_error = msg;
    return code;
}

template <typename T>
int dalloc(sllm_engine* e, T** p, size_t count, uint64_t* counter) {
    void* q = nullptr;
    const size_t bytes = std::max<size_t>(count * sizeof(T), 256);
    CU(cudaMalloc(&q, bytes));
    CU(cudaMemsetAsync(q, 0, bytes, e->stream));
    e->allocs.push_back(q);
    *p = static_cast<T*>(q);
    if (counter) *counter += bytes;
    return SLLM_OK;
}

size_t wsize(const sllm_engine* e) { return e->f32 ? 4 : 2; }

// ---- launch helper: every kernel of the engine goes through here ---------------------------------
template <typename... KArgs, typename... Args>
int launch(sllm_engine* e, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, bool pdl, Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = e->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
    CU(cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...));
    e->launches += 1;
    return SLLM_OK;
}

// Dynamic shared memory above 48 KB is opted into once, at engine creation (configure_kernels).
template <typename K>
int set_smem(sllm_engine*, K, size_t) { return SLLM_OK; }

template <typename K>
int opt_in_smem(sllm_engine* e, K kern) {
    // the opt-in limit covers static + dynamic shared memory of the kernel
    cudaFuncAttributes fa{};
    CU(cudaFuncGetAttributes(&fa, kern));
    CU(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                            (int)(e->max_dyn_smem - fa.sharedSizeBytes)));
    return SLLM_OK;
}

// ---- projections ---------------------------------------------------------------------------------------
template <typename WT, int MODE, int PF>
int launch_gemv_pf(sllm_engine* e, const GemvArgs& a, bool pdl, int nt, dim3 grid, size_t smem) {
    switch (nt) {
        case 1: return launch(e, k_gemv<WT, 1, MODE, PF>, grid, dim3(kGemvThreads), smem, pdl, a);
        case 2: return launch(e, k_gemv<WT, 2, MODE, PF>, grid, dim3(kGemvThreads), smem, pdl, a);
        case 4: return launch(e, k_gemv<WT, 4, MODE, PF>, grid, dim3(kGemvThreads), smem, pdl, a);
        default: return launch(e, k_gemv<WT, 8, MODE, PF>, grid, dim3(kGemvThreads), smem, pdl, a);
    }
}

template <typename WT, int MODE>
int launch_gemv(sllm_engine* e, GemvArgs a, bool pdl) {
    const int groups = a.R / 2;
    int gx = std::min((groups + kGemvWarps - 1) / kGemvWarps, e->sm_count * (a.prenorm ? 16 : 4));
    const int n = a.n_tok;
    int nt = n == 1 ? 1 : (n == 2 ? 2 : (n <= 4 ? 4 : 8));
    const size_t smem = (size_t)nt * a.K * sizeof(float);
    if (smem + 1024 > e->max_dyn_smem) return fail(e, SLLM_ERR_INVALID, "projection input does not fit shared memory");
    const dim3 grid(gx, (n + nt - 1) / nt);
    // register prefetch depth: 3 chunks per lane cover K = 640 in bf16, 7 cover K = 1728
    const int chunks_per_lane = (a.K / Elems<WT>::per16 + 31) / 32;
    if (chunks_per_lane > 3) return launch_gemv_pf<WT, MODE, 7>(e, a, pdl, nt, grid, smem);
    return launch_gemv_pf<WT, MODE, 3>(e, a, pdl, nt, grid, smem);
}

template <typename KVT, int HD>
int launch_attn_stream_hd(sllm_engine* e, const AttnDecArgs& a, bool pdl) {
    return launch(e, k_attn_stream<KVT, HD, kStreamStages>, dim3(a.n_splits, a.m.H, a.pass.n_tok), dim3(kStreamThreads),
                  attn_stream_smem<KVT, HD, kStreamStages>(), pdl, a, e->d_status);
}

template <typename KVT, int HD>
int launch_attn_prefill_hd(sllm_engine* e, const AttnDecArgs& a, bool pdl) {
    AttnPfArgs p{};
    p.q = a.q; p.out = a.out; p.out_bf16 = a.out_bf16; p.m = a.m; p.kv = a.kv; p.tiles = a.pass.tiles; p.layer = a.layer;
    p.status = e->d_status;
    return launch(e, k_attn_prefill<KVT, HD>, dim3(a.pass.n_tiles, a.m.H), dim3(kPfThreads), attn_prefill_smem<KVT, HD>(), pdl, p);
}

template <typename KVT>
int launch_attn(sllm_engine* e, const AttnDecArgs& a, bool pdl) {
    if (a.pass.n_tiles > 0 && a.pass.n_tiles * 4 <= a.pass.n_tok) {      // long runs of one sequence: query tiles share the pages
        if (e->attn_tc && sizeof(KVT) == 2) {
            AttnPtArgs p{};
            p.q = a.q; p.out = a.out; p.out_bf16 = a.out_bf16; p.m = a.m; p.kv = a.kv; p.tiles = a.pass.tiles; p.layer = a.layer;
            p.status = e->d_status;
            return launch(e, k_attn_prefill_tc, dim3(a.pass.n_tiles, a.m.H), dim3(kPtThreads), attn_prefill_tc_smem(), pdl, e->map_kv, p);
        }
        switch (a.m.hd) {
            case 16: return launch_attn_prefill_hd<KVT, 16>(e, a, pdl);
            case 32: return launch_attn_prefill_hd<KVT, 32>(e, a, pdl);
            case 64: return launch_attn_prefill_hd<KVT, 64>(e, a, pdl);
            case 128: return launch_attn_prefill_hd<KVT, 128>(e, a, pdl);
        }
    }
    if ((a.prefer_stream || a.n_splits == 1 || a.pass.n_tok * a.m.H >= e->sm_count) && e->use_attn_stream) {   // stream pages through shared memory
        switch (a.m.hd) {
            case 16: return launch_attn_stream_hd<KVT, 16>(e, a, pdl);
            case 32: return launch_attn_stream_hd<KVT, 32>(e, a, pdl);
            case 64: return launch_attn_stream_hd<KVT, 64>(e, a, pdl);
            case 128: return launch_attn_stream_hd<KVT, 128>(e, a, pdl);
        }
    }
    const dim3 grid(a.n_splits, a.m.H, a.pass.n_tok), block(kAttnThreads);
    switch (a.m.hd) {
        case 16: return launch(e, k_attn_decode<KVT, 16>, grid, block, 0, pdl, a);
        case 32: return launch(e, k_attn_decode<KVT, 32>, grid, block, 0, pdl, a);
        case 64: return launch(e, k_attn_decode<KVT, 64>, grid, block, 0, pdl, a);
        case 128: return launch(e, k_attn_decode<KVT, 128>, grid, block, 0, pdl, a);
    }
    return fail(e, SLLM_ERR_INVALID, "unsupported head_dim");
}

// Runs the model over the pass's token list.  Logits are produced for n_rows rows
// (row_tok[i] = pass-token index, NULL = identity) into `logits`.
template <typename WT>
int run_pass_t(sllm_engine* e, const PassView& pv, const int* row_tok, int n_rows, float* logits, bool pdl) {
    const ModelDims& m = e->md;
    KvView kv{e->kv_pool, e->d_block_table, e->n_pages, e->pages_per_seq};
    const int n = pv.n_tok;
    // attention split policy: fill the GPU when few (token, head) pairs exist
    int n_splits = 1, kps = ((m.ctx + kPage - 1) / kPage) * kPage;
    if (pv.n_tiles == 0 && n <= e->split_tok_cap && n * m.H < 2 * e->sm_count) {
        n_splits = std::min({kMaxSplits, e->pages_per_seq, std::max(1, 4 * e->sm_count / (n * m.H))});
        const int pages_per_split = (e->pages_per_seq + n_splits - 1) / n_splits;
        kps = pages_per_split * kPage;
        n_splits = (e->pages_per_seq + pages_per_split - 1) / pages_per_split;
    }
    for (int l = 0; l < m.L; ++l) {
        const LayerW& w = e->layers[l];
        GemvArgs a{};
        a.m = m; a.kv = kv; a.pass = pv; a.layer = l; a.rope = e->rope; a.eps = m.eps; a.n_tok = n;
        // QKV (+ embedding gather on layer 0)
        a.W = w.wqkv; a.R = 3 * m.D; a.K = m.D; a.in = e->x; a.gain = w.g_attn; a.out = e->q;
        a.emb = (l == 0) ? e->emb_f32 : nullptr; a.x_out = e->x;
        int rc = launch_gemv<WT, kModeQKV>(e, a, pdl);
        if (rc) return rc;
        AttnDecArgs t{};
        t.q = e->q; t.out = e->att; t.m = m; t.kv = kv; t.pass = pv; t.layer = l;
        t.n_splits = n_splits; t.keys_per_split = kps;
        t.part_o = e->part_o; t.part_ml = e->part_ml; t.ticket = e->ticket;
        rc = launch_attn<WT>(e, t, pdl);
        if (rc) return rc;
        a.emb = nullptr;
        a.W = w.wo; a.R = m.D; a.K = m.D; a.in = e->att; a.out = e->x;
        rc = launch_gemv<WT, kModeResidual>(e, a, pdl);
        if (rc) return rc;
        a.W = w.wgu; a.R = 2 * m.F; a.K = m.D; a.in = e->x; a.gain = w.g_ffn; a.out = e->hid;
        rc = launch_gemv<WT, kModeGateUp>(e, a, pdl);
        if (rc) return rc;
        a.W = w.wd; a.R = m.D; a.K = m.F; a.in = e->hid; a.out = e->x;
        rc = launch_gemv<WT, kModeResidual>(e, a, pdl);
        if (rc) return rc;
    }
    if (n_rows > 0) {
        GemvArgs a{};
        a.m = m; a.eps = m.eps; a.W = e->emb_w; a.R = m.V; a.K = m.D; a.in = e->x; a.gain = e->g_final;
        a.out = logits; a.n_tok = n_rows; a.row_tok = row_tok; a.pass = pv;
        int rc = launch_gemv<WT, kModeHead>(e, a, pdl);
        if (rc) return rc;
    }
    return SLLM_OK;
}


// ---- tensor-core path: tensor maps and launches ------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// bf16 matrix [rows][K] (K contiguous) -> map with boxes of 64 x box_rows elements, 128-byte swizzle
int make_map(sllm_engine* e, CUtensorMap* map, const void* base, uint64_t rows, uint64_t K, uint32_t box_rows) {
    const cuuint64_t gdim[2] = {K, rows};
    const cuuint64_t gstride[1] = {K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kTcBK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = reinterpret_cast<EncodeTiledFn>(e->encode_tiled)(
        map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstride, box, estr,
        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(e, SLLM_ERR_CUDA, "cuTensorMapEncodeTiled failed (" + std::to_string((int)r) + ")");
    return SLLM_OK;
}

int x_map(sllm_engine* e, const void* buf, uint64_t rows_cap, uint64_t K, int bn, CUtensorMap* out) {
    auto key = std::make_pair(buf, bn);
    auto it = e->map_x.find(key);
    if (it == e->map_x.end()) {
        CUtensorMap m;
        int rc = make_map(e, &m, buf, rows_cap, K, (uint32_t)bn);
        if (rc) return rc;
        it = e->map_x.emplace(key, m).first;
    }
    *out = it->second;
    return SLLM_OK;
}

int pick_split(const sllm_engine* e, int bn, int tiles, int nkb, bool wide);

template <int BN, int MODE>
int launch_tc_bn(sllm_engine* e, const CUtensorMap& mw, const CUtensorMap& mx, TcArgs a, bool pdl) {
    const int tiles = ((a.R + kTcBM - 1) / kTcBM) * ((a.n_tok + BN - 1) / BN);
    const int nkb = (a.K + kTcBK - 1) / kTcBK;
    // the transposing epilogue (16-byte accesses need every row count to be a multiple of 4)
    const bool wide = a.R % 4 == 0 && a.m.D % 4 == 0 && a.m.hd % 4 == 0 && !e->tune_no_wide_epi;
    // split-K over a cluster while the tiles alone leave most SMs idle
    const int split = pick_split(e, BN, tiles, nkb, wide);
    const int kb_per_block = (nkb + split - 1) / split;
    a.wide_epi = wide ? 1 : 0;
    const int fit = (int)((e->max_dyn_smem - tc_fixed_bytes(BN, split, wide)) / tc_stage_bytes(BN));
    a.split = split;
    const int cap = BN >= 256 ? 4 : (BN >= 128 ? 6 : (BN >= 64 ? 8 : 10));   // beyond this, measured slower (less room for the next kernel's blocks)
    a.stages = std::max(1, std::min({cap, fit, kb_per_block}));
    // more than one wave of tiles: one block per SM walks its tiles with two accumulators (see TcArgs)
    a.n_tiles = tiles;
    a.persistent = (split == 1 && 2 * BN <= 512 && tiles > e->sm_count && !e->tune_no_persistent_tc) ? 1 : 0;
    const dim3 grid = a.persistent ? dim3(std::min(tiles, e->sm_count))
                                   : dim3((a.R + kTcBM - 1) / kTcBM, (a.n_tok + BN - 1) / BN, split);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = dim3(tc_threads<BN>()); cfg.dynamicSmemBytes = tc_smem_bytes(BN, a.stages, split, wide); cfg.stream = e->stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (split > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 1; attr[na].val.clusterDim.y = 1; attr[na].val.clusterDim.z = split;
        ++na;
    }
    if (pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr; cfg.numAttrs = na;
    CU(cudaLaunchKernelEx(&cfg, k_gemm_tc<BN, MODE>, mw, mx, a));
    e->launches += 1;
    return SLLM_OK;
}

// split-K cluster size for `tiles` tiles of width bn over nkb K blocks: about 3 K blocks per block at least, no more
// blocks than SMs, and the peers' accumulators must fit block 0's shared memory
int pick_split(const sllm_engine* e, int bn, int tiles, int nkb, bool wide) {
    int split = std::min({kTcMaxSplit, std::max(1, nkb / 3), std::max(1, e->sm_count / tiles)});
    // A cluster's blocks must sit in one GPC (18 or 19 SMs of this chip's 148): clusters of 7 fit twice per GPC, so 20
    // tiles dealt 7 ways (140 blocks) run in two rounds where clusters of 6 (three per GPC) run in one -- measured
    // 1.52 against 1.44 ms per iteration at 128 sequences.  Keep every cluster resident at once.
    const int gpcs = std::max(1, e->sm_count / 18);
    while (split > 1 && tiles > gpcs * (18 / split)) --split;
    if (e->tune_tc_split > 0) split = std::min({e->tune_tc_split, kTcMaxSplit, nkb});
    while (split > 1 && tc_smem_bytes(bn, 2, split, wide) > e->max_dyn_smem) --split;
    return split;
}

// token-tile width: wide tiles for arithmetic intensity, narrower ones while the grid would not fill the GPU
int pick_bn(const sllm_engine* e, int R, int n, int K) {
    const int tiles_m = (R + kTcBM - 1) / kTcBM;
    if (n <= 32) return 32;
    if (n <= 64) return tiles_m * 2 <= e->sm_count ? 32 : 64;      // small projections: two token tiles, twice the blocks
    // the widest token tile that still gives at least half an SM count of blocks: wide tiles re-read the
    // weight tile less often (shared-memory fill traffic from L2 is what bounds these small-K products)
    for (int bn : {256, 128, 64}) if (tiles_m * ((n + bn - 1) / bn) * 2 >= e->sm_count) return bn;
    // Few row tiles (the residual projections): a block of a 32-token tile takes in (128 + 32) x K x 2 bytes, and one
    // SM's intake (~65 GB/s) is what its time is made of when K is large (the down projection: 553 KB).  64-token
    // tiles with the K blocks dealt over a cluster move fewer bytes per SM; the hand-over between the cluster's blocks
    // costs about as much as 100 KB of intake.  Taken when clearly ahead (measured: 4.19 -> 4.16 ms per iteration at
    // 512 sequences, where the model says 0.58; 3.237 -> 3.247 at 384, where it says 0.71).
    const int nkb = (K + kTcBK - 1) / kTcBK;
    auto cost = [&](int bn) {
        const int split = pick_split(e, bn, tiles_m * ((n + bn - 1) / bn), nkb, true);
        return (double)(kTcBM + bn) * K * 2.0 / split + (split > 1 ? 100e3 : 0.0);
    };
    return cost(64) < 0.65 * cost(32) ? 64 : 32;
}

template <int MODE>
int launch_tc(sllm_engine* e, const CUtensorMap& mw, const void* xbuf, uint64_t x_rows_cap, const TcArgs& a, bool pdl) {
    const int bn = pick_bn(e, a.R, a.n_tok, a.K);
    CUtensorMap mx;
    int rc = x_map(e, xbuf, x_rows_cap, (uint64_t)a.K, bn, &mx);
    if (rc) return rc;
    switch (bn) {
        case 32: return launch_tc_bn<32, MODE>(e, mw, mx, a, pdl);
        case 64: return launch_tc_bn<64, MODE>(e, mw, mx, a, pdl);
        case 128: return launch_tc_bn<128, MODE>(e, mw, mx, a, pdl);
        default: return launch_tc_bn<256, MODE>(e, mw, mx, a, pdl);
    }
}

template <int MODE>
int configure_tc(sllm_engine* e) {
    int rc = SLLM_OK;
    auto set = [&](auto kern, size_t bytes) {
        if (!rc && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess)
            rc = fail(e, SLLM_ERR_CUDA, "cudaFuncSetAttribute failed for the tensor-core projection kernel");
    };
    set(k_gemm_tc<32, MODE>, e->max_dyn_smem);
    set(k_gemm_tc<64, MODE>, e->max_dyn_smem);
    set(k_gemm_tc<128, MODE>, e->max_dyn_smem);
    set(k_gemm_tc<256, MODE>, e->max_dyn_smem);
    return rc;
}

int launch_attn_any(sllm_engine* e, const AttnDecArgs& t, bool pdl);

// The model over a pass of many tokens, bf16 weights: tcgen05 projections.
int run_pass_tc(sllm_engine* e, const PassView& pv, const int* row_tok, int n_rows, float* logits, bool pdl) {
    const ModelDims& m = e->md;
    KvView kv{e->kv_pool, e->d_block_table, e->n_pages, e->pages_per_seq};
    const int n = pv.n_tok;
    TcArgs a{};
    a.m = m; a.kv = kv; a.pass = pv; a.rope = e->rope; a.status = e->d_status; a.n_tok = n;
    for (int l = 0; l < m.L; ++l) {
        const LayerW& w = e->layers[l];
        a.layer = l;
        // RMSNorm is folded into the projections (TcArgs): only the first layer needs a kernel of its own, which
        // also gathers the embedding rows
        int rc = SLLM_OK;
        if (l == 0) {
            rc = launch(e, k_embed_prep, dim3(n), dim3(256), 0, pdl, (const float*)e->emb_f32, pv.tok_id, w.g_attn, e->x, e->xn16,
                        e->ss_part, m.D, e->ss_parts);
            if (rc) return rc;
        }
        a.ss_in = e->ss_part; a.n_parts = e->ss_parts; a.eps = m.eps;
        a.gain_next = nullptr; a.xn_out = nullptr; a.ss_out = nullptr;
        a.R = 3 * m.D; a.K = m.D; a.out = e->q; a.out_bf16 = nullptr;
        rc = launch_tc<kModeQKV>(e, e->map_wqkv[l], e->xn16, e->pass_cap, a, pdl);
        if (rc) return rc;
        AttnDecArgs t{};
        t.q = e->q; t.out = e->att; t.out_bf16 = e->att16; t.m = m; t.kv = kv; t.pass = pv; t.layer = l;
        {
            const int pairs = n * m.H;
            t.n_splits = 1;
            t.keys_per_split = e->pages_per_seq * kPage;
            if (pv.n_tiles == 0 && n <= e->split_tok_cap && pairs < 4 * e->sm_count) {
                // the streaming kernel: split each pair's pages over several blocks, about 8 blocks per SM in all
                // (measured at 32 and 64 sequences: 4 splits and 1 split are the fastest; at 8 sequences 8 splits);
                // none once the pairs alone fill the 4 resident blocks per SM
                t.n_splits = std::max(1, std::min(pairs < e->sm_count ? 8 : 4, (8 * e->sm_count + pairs / 2) / pairs));
                t.prefer_stream = 1;
            }
        }
        if (e->tune_stream_splits > 0 && pv.n_tiles == 0 && n <= e->split_tok_cap) t.n_splits = e->tune_stream_splits;
        t.part_o = e->part_o; t.part_ml = e->part_ml; t.ticket = e->ticket;
        rc = launch_attn_any(e, t, pdl);
        if (rc) return rc;
        a.R = m.D; a.K = m.D; a.out = e->x;
        a.ss_in = nullptr; a.gain_next = w.g_ffn; a.xn_out = e->xn16; a.ss_out = e->ss_part;
        rc = launch_tc<kModeResidual>(e, e->map_wo[l], e->att16, e->pass_cap, a, pdl);
        if (rc) return rc;
        a.ss_in = e->ss_part; a.gain_next = nullptr; a.xn_out = nullptr; a.ss_out = nullptr;
        a.R = 2 * m.F; a.K = m.D; a.out = nullptr; a.out_bf16 = e->hid16;
        rc = launch_tc<kModeGateUp>(e, e->map_wgu[l], e->xn16, e->pass_cap, a, pdl);
        if (rc) return rc;
        a.R = m.D; a.K = m.F; a.out = e->x; a.out_bf16 = nullptr;
        a.ss_in = nullptr;
        if (l + 1 < m.L) { a.gain_next = e->layers[l + 1].g_attn; a.xn_out = e->xn16; a.ss_out = e->ss_part; }
        rc = launch_tc<kModeResidual>(e, e->map_wd[l], e->hid16, e->pass_cap, a, pdl);
        if (rc) return rc;
    }
    if (n_rows > 0) {
        if (n_rows > e->logit_rows_cap) return fail(e, SLLM_ERR_INVALID, "too many logits rows for one pass");
        int rc = launch(e, k_rmsnorm_bf16, dim3(n_rows), dim3(256), 0, pdl, (const float*)e->x, (const float*)e->g_final,
                        e->head16, m.D, m.eps, row_tok, (const float*)nullptr, pv.tok_id, e->x);
        if (rc) return rc;
        TcArgs h = a;
        h.R = m.V; h.K = m.D; h.out = logits; h.out_bf16 = nullptr; h.n_tok = n_rows;
        rc = launch_tc<kModeHead>(e, e->map_head, e->head16, e->logit_rows_cap, h, pdl);
        if (rc) return rc;
    }
    return SLLM_OK;
}


// ---- fused single-token decode path (decode_fused.cuh) ------------------------------------------------------
template <typename... KArgs>
int launch_cluster(sllm_engine* e, void (*kern)(KArgs...), dim3 grid, size_t smem, bool pdl, const FusedArgs& a) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = dim3(kFusedThreads); cfg.dynamicSmemBytes = smem; cfg.stream = e->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kCS; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = pdl ? 2 : 1;
    CU(cudaLaunchKernelEx(&cfg, kern, a));
    e->launches += 1;
    return SLLM_OK;
}

template <typename WT, int PF>
int launch_attn_block(sllm_engine* e, const FusedArgs& a, bool pdl) {
    const dim3 grid(kCS, a.m.H);
    const size_t smem = (size_t)3 * a.m.D * sizeof(float);
    switch (a.m.hd) {
        case 16: return launch_cluster(e, k_attn_block<WT, 16, PF>, grid, smem, pdl, a);
        case 32: return launch_cluster(e, k_attn_block<WT, 32, PF>, grid, smem, pdl, a);
        case 64: return launch_cluster(e, k_attn_block<WT, 64, PF>, grid, smem, pdl, a);
        case 128: return launch_cluster(e, k_attn_block<WT, 128, PF>, grid, smem, pdl, a);
    }
    return fail(e, SLLM_ERR_INVALID, "unsupported head_dim");
}

template <typename WT>
int run_pass_fused_t(sllm_engine* e, const PassView& pv, int n_rows, float* logits, bool pdl) {
    const ModelDims& m = e->md;
    const int chunks_per_lane = (m.D / Elems<WT>::per16 + 31) / 32;
    const int G = kFusedThreads / (m.D / Elems<WT>::per16);
    const size_t smem_b = (size_t)(2 + std::max(G, 2)) * m.D * sizeof(float);      // xs | group sums | receive buffer
    const int ncl = e->fused_nb / kCS;
    FusedArgs a{};
    a.m = m; a.kv = KvView{e->kv_pool, e->d_block_table, e->n_pages, e->pages_per_seq};
    a.tok_id = pv.tok_id; a.tok_slot = pv.tok_slot; a.tok_pos = pv.tok_pos; a.rope = e->rope; a.upc = e->fused_upc;
    for (int l = 0; l < m.L; ++l) {
        const LayerW& w = e->layers[l];
        a.layer = l;
        // attention block: reads xb + down partials of the previous layer (layer 0: the embedding row), writes x
        a.x_in = e->xb; a.parts_in = e->down_parts; a.n_parts_in = l == 0 ? 0 : ncl; a.x_out = e->x;
        a.emb = l == 0 ? e->emb_f32 : nullptr; a.gain = w.g_attn; a.w1 = w.wqkv; a.w2 = w.wo; a.parts_out = e->attn_parts;
        int rc = chunks_per_lane > 3 ? launch_attn_block<WT, 7>(e, a, pdl) : launch_attn_block<WT, 3>(e, a, pdl);
        if (rc) return rc;
        // FFN block: reads x + attention partials, writes xb
        a.x_in = e->x; a.parts_in = e->attn_parts; a.n_parts_in = m.H; a.x_out = e->xb; a.emb = nullptr;
        a.gain = w.g_ffn; a.w1 = w.wgu; a.w2 = e->wdT[l]; a.parts_out = e->down_parts;
        rc = chunks_per_lane > 3 ? launch_cluster(e, k_ffn_block<WT, 7>, dim3(e->fused_nb), smem_b, pdl, a)
                                 : launch_cluster(e, k_ffn_block<WT, 3>, dim3(e->fused_nb), smem_b, pdl, a);
        if (rc) return rc;
    }
    if (n_rows > 0) {
        int rc = launch(e, k_final_norm, dim3(1), dim3(kFusedThreads), (size_t)3 * m.D * sizeof(float), pdl, (const float*)e->xb,
                        (const float*)e->down_parts, ncl, m.D, (const float*)e->g_final, m.eps, e->q);
        if (rc) return rc;
        GemvArgs h{};
        h.m = m; h.eps = m.eps; h.W = e->emb_w; h.R = m.V; h.K = m.D; h.in = e->q; h.gain = e->g_final; h.prenorm = 1;
        h.out = logits; h.n_tok = 1; h.pass = pv;
        return launch_gemv<WT, kModeHead>(e, h, pdl);
    }
    // no logits wanted: leave the finished residual in e->x, where the other paths keep it
    return launch(e, k_sum_parts, dim3((m.D + 255) / 256), dim3(256), 0, pdl, (const float*)e->xb, (const float*)e->down_parts,
                  ncl, m.D, e->x);
}

int launch_attn_any(sllm_engine* e, const AttnDecArgs& t, bool pdl) { return launch_attn<__nv_bfloat16>(e, t, pdl); }

template <int HD>
int launch_persist_hd(sllm_engine* e, const PersistArgs& a, bool pdl) {
    return launch(e, k_decode_persist<HD>, dim3(a.na), dim3(kPsBlock), e->ps_smem, pdl, a);
}

// One token through every layer and the head as a single resident kernel.
int run_pass_persist(sllm_engine* e, const PassView& pv, int n_rows, float* logits, bool pdl, const SampleArgs* fold) {
    PersistArgs a{};
    a.fold_temperature = -1.f;
    if (fold && n_rows > 0) {                                   // the next sampling step's first two kernels ride along
        a.fold_temperature = fold->temperature > 0.f ? fold->temperature : 0.f;
        a.fold_penalty = fold->penalty; a.st = fold->st;
        a.g_mass = fold->g_mass; a.g_cnt = fold->g_cnt; a.g_w = fold->g_w; a.g_pmax_val = fold->g_pmax_val; a.g_pmax_idx = fold->g_pmax_idx;
        a.mxb = e->ps_mxb;
    }
    a.m = e->md; a.kv = KvView{e->kv_pool, e->d_block_table, e->n_pages, e->pages_per_seq};
    a.tok_id = pv.tok_id; a.tok_slot = pv.tok_slot; a.tok_pos = pv.tok_pos;
    a.layers = e->d_layers; a.emb_f32 = e->emb_f32; a.emb_w = static_cast<const __nv_bfloat16*>(e->emb_w);
    a.g_final = e->g_final; a.rope = e->rope;
    a.xa = e->ps_xa; a.xb = e->ps_xb; a.qkv = e->ps_qkv; a.ap = e->ps_ap; a.hb = e->ps_hb;
    a.epoch = e->ps_epoch; a.status = e->d_status;
    a.logits = n_rows > 0 ? logits : nullptr; a.x_out = e->x;
    a.na = e->ps_na; a.s_max = e->ps_smax; a.pps_max = e->ps_ppsmax; a.smem_total = (uint32_t)e->ps_smem;
    switch (e->md.hd) {
        case 16: return launch_persist_hd<16>(e, a, pdl);
        case 32: return launch_persist_hd<32>(e, a, pdl);
        case 64: return launch_persist_hd<64>(e, a, pdl);
        case 128: return launch_persist_hd<128>(e, a, pdl);
    }
    return fail(e, SLLM_ERR_INVALID, "unsupported head_dim");
}

// Whether a decode pass over the live slots would run as the persistent single-token kernel (which can carry the next
// sampling step's first two kernels).
bool pass_is_persistent(const sllm_engine* e, int n_tok) { return n_tok == 1 && e->persist_ok; }

int run_pass(sllm_engine* e, const PassView& pv, const int* row_tok, int n_rows, float* logits, bool pdl, const SampleArgs* fold = nullptr) {
    if (pass_is_persistent(e, pv.n_tok) && (n_rows == 0 || row_tok == nullptr)) return run_pass_persist(e, pv, n_rows, logits, pdl, fold);
    if (pv.n_tok == 1 && e->fused_ok && (n_rows == 0 || row_tok == nullptr))
        return e->f32 ? run_pass_fused_t<float>(e, pv, n_rows, logits, pdl) : run_pass_fused_t<__nv_bfloat16>(e, pv, n_rows, logits, pdl);
    if (!e->f32 && e->encode_tiled && pv.n_tok >= e->tc_min_tokens) return run_pass_tc(e, pv, row_tok, n_rows, logits, pdl);
    return e->f32 ? run_pass_t<float>(e, pv, row_tok, n_rows, logits, pdl)
                  : run_pass_t<__nv_bfloat16>(e, pv, row_tok, n_rows, logits, pdl);
}

template <typename WT, int MODE>
int configure_gemv(sllm_engine* e) {
    int rc = opt_in_smem(e, k_gemv<WT, 1, MODE, 3>);
    if (!rc) rc = opt_in_smem(e, k_gemv<WT, 2, MODE, 3>);
    if (!rc) rc = opt_in_smem(e, k_gemv<WT, 4, MODE, 3>);
    if (!rc) rc = opt_in_smem(e, k_gemv<WT, 8, MODE, 3>);
    if (!rc) rc = opt_in_smem(e, k_gemv<WT, 1, MODE, 7>);
    if (!rc) rc = opt_in_smem(e, k_gemv<WT, 2, MODE, 7>);
    if (!rc) rc = opt_in_smem(e, k_gemv<WT, 4, MODE, 7>);
    if (!rc) rc = opt_in_smem(e, k_gemv<WT, 8, MODE, 7>);
    return rc;
}
template <typename WT>
int configure_kernels_t(sllm_engine* e) {
    auto big = [&](auto kern, size_t bytes) -> int {
        CU(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
        return SLLM_OK;
    };
    int rc = big(k_attn_prefill<WT, 16>, attn_prefill_smem<WT, 16>());
    if (!rc) rc = big(k_attn_prefill<WT, 32>, attn_prefill_smem<WT, 32>());
    if (!rc) rc = big(k_attn_prefill<WT, 64>, attn_prefill_smem<WT, 64>());
    if (!rc) rc = big(k_attn_prefill<WT, 128>, attn_prefill_smem<WT, 128>());
    if (!rc) rc = big(k_attn_stream<WT, 16, kStreamStages>, attn_stream_smem<WT, 16, kStreamStages>());
    if (!rc) rc = big(k_attn_stream<WT, 32, kStreamStages>, attn_stream_smem<WT, 32, kStreamStages>());
    if (!rc) rc = big(k_attn_stream<WT, 64, kStreamStages>, attn_stream_smem<WT, 64, kStreamStages>());
    if (!rc) rc = big(k_attn_stream<WT, 128, kStreamStages>, attn_stream_smem<WT, 128, kStreamStages>());
    if (rc) return rc;
    rc = configure_gemv<WT, kModeQKV>(e);
    if (!rc) rc = configure_gemv<WT, kModeResidual>(e);
    if (!rc) rc = configure_gemv<WT, kModeGateUp>(e);
    if (!rc) rc = configure_gemv<WT, kModeHead>(e);
    return rc;
}
int configure_kernels(sllm_engine* e);

// ---- KV pages ------------------------------------------------------------------------------------------
int ensure_pages(sllm_engine* e, int slot, int n_positions, bool* changed) {
    const int need = (std::min(n_positions, e->md.ctx) + kPage - 1) / kPage;
    auto& pages = e->slot_pages[slot];
    while ((int)pages.size() < need) {
        if (e->free_pages.empty()) return fail(e, SLLM_ERR_CAPACITY, "KV page pool exhausted");
        pages.push_back(e->free_pages.back());
        e->free_pages.pop_back();
        *changed = true;
    }
    return SLLM_OK;
}

int upload_block_table(sllm_engine* e, int slot) {
    const auto& pages = e->slot_pages[slot];
    if (pages.empty()) return SLLM_OK;
    CU(cudaMemcpyAsync(e->d_block_table + (size_t)slot * e->pages_per_seq, pages.data(), pages.size() * sizeof(int),
                       cudaMemcpyHostToDevice, e->stream));
    return SLLM_OK;
}

void release_slot(sllm_engine* e, int slot) {
    for (int p : e->slot_pages[slot]) e->free_pages.push_back(p);
    e->slot_pages[slot].clear();
    e->h_len_bound[slot] = 0;
}

int sampling_check(sllm_engine* e, const sllm_sampling* o) {
    if (!o) return fail(e, SLLM_ERR_INVALID, "sampling options missing");
    if (o->temperature > 0.0f && !(o->top_p == o->top_p)) return fail(e, SLLM_ERR_INVALID, "top_p is NaN");
    if (o->repetition_penalty == 0.0f) return fail(e, SLLM_ERR_INVALID, "repetition_penalty must be non-zero");
    return SLLM_OK;
}

SampleArgs make_sample_args(sllm_engine* e, const sllm_sampling* o, int n_slots, const double* d_draws, int stride,
                            int seeded) {
    SampleArgs s{};
    s.logits = e->step_logits; s.st = e->st; s.V = e->md.V; s.ctx = e->md.ctx;
    s.temperature = o->temperature; s.top_p = o->top_p; s.penalty = o->repetition_penalty;
    s.eos = o->eos_token; s.stop_token = o->stop_token;
    s.draws = d_draws; s.n_slots = n_slots; s.draws_stride = stride; s.seeded = seeded;
    s.g_mass = e->samp_mass; s.g_cnt = e->samp_cnt; s.g_w = e->samp_w; s.g_pmax_val = e->samp_pmax_val; s.g_pmax_idx = e->samp_pmax_idx;
    // blocks per slot of the two partial kernels: spread one slot over the GPU, many slots one block row each
    s.bps = std::max(1, std::min(e->samp_bps_cap, (2 * e->sm_count) / std::max(1, n_slots)));
    s.next_tok_id = e->d_dec_id; s.next_tok_pos = e->d_dec_pos; s.next_tok_slot = e->d_dec_slot;
    return s;
}

int configure_kernels(sllm_engine* e) {
    // static shared memory of the sampler (histograms) counts against the same limit
    cudaFuncAttributes fa{};
    CU(cudaFuncGetAttributes(&fa, k_samp_pick));
    CU(cudaFuncSetAttribute(k_samp_pick, cudaFuncAttributeMaxDynamicSharedMemorySize,
                            (int)(e->max_dyn_smem - fa.sharedSizeBytes)));
    if ((size_t)e->md.V * sizeof(float) + fa.sharedSizeBytes > e->max_dyn_smem)
        return fail(e, SLLM_ERR_INVALID, "vocab_size does not fit the sampler's shared memory");
    return e->f32 ? configure_kernels_t<float>(e) : configure_kernels_t<__nv_bfloat16>(e);
}

// folded: the persistent decode kernel before this sampling step has already produced the per-part maxima (one part
// per block of its grid), the weights and the level-0 histogram: only the pick kernel is left.
int launch_sampler(sllm_engine* e, SampleArgs s, bool pdl, bool folded = false) {
    int rc = SLLM_OK;
    if (folded) {
        s.bps = e->ps_na;
    } else {
        const dim3 part_grid(s.bps, s.n_slots);
        rc = launch(e, k_samp_max, part_grid, dim3(kSampPartThreads), 0, pdl, s);
        if (rc) return rc;
        if (s.temperature > 0.0f) {
            rc = launch(e, k_samp_hist, part_grid, dim3(kSampPartThreads), 0, pdl, s);
            if (rc) return rc;
        }
    }
    const size_t smem = s.temperature > 0.0f ? (size_t)e->md.V * sizeof(float) : 16;
    return launch(e, k_samp_pick, dim3(s.n_slots), dim3(kSampThreads), smem, pdl, s);
}

// host bound on lengths: one more token per live slot per sampling step
int grow_for_step(sllm_engine* e) {
    for (int s = 0; s < e->n_live; ++s) {
        if (e->slot_released[s]) continue;
        bool changed = false;
        e->h_len_bound[s] = std::min(e->h_len_bound[s] + 1, e->md.ctx + 1);
        int rc = ensure_pages(e, s, e->h_len_bound[s], &changed);
        if (rc) return rc;
        if (changed) { rc = upload_block_table(e, s); if (rc) return rc; }
    }
    return SLLM_OK;
}

// With more (token, head) blocks than the GPU holds at once, the attention kernel's last blocks to start should be
// its shortest: the decode pass hands it the slots sorted by descending length.
bool decode_uses_order(const sllm_engine* e) { return e->n_live * e->md.H >= e->order_min_waves * 4 * e->sm_count; }

PassView decode_view(sllm_engine* e) {
    return PassView{e->d_dec_id, e->d_dec_slot, e->d_dec_pos, e->n_live, nullptr, 0,
                    decode_uses_order(e) ? e->d_attn_order : nullptr};
}

// Lengths grow in step, so the order computed from the host's bounds stays right for a whole run of iterations;
// it is a scheduling hint only (any permutation gives the same results).
int refresh_attn_order(sllm_engine* e) {
    if (!decode_uses_order(e)) return SLLM_OK;
    e->h_attn_order.resize(e->n_live);
    for (int i = 0; i < e->n_live; ++i) e->h_attn_order[i] = i;
    std::stable_sort(e->h_attn_order.begin(), e->h_attn_order.end(),
                     [&](int x, int y) { return e->h_len_bound[x] > e->h_len_bound[y]; });
    CU(cudaMemcpyAsync(e->d_attn_order, e->h_attn_order.data(), (size_t)e->n_live * sizeof(int), cudaMemcpyHostToDevice, e->stream));
    CU(cudaStreamSynchronize(e->stream));           // the host vector may change before the copy would otherwise run
    return SLLM_OK;
}

// One decode iteration = sampler, then the model over the sampled tokens.  fold_in: the pass before this iteration
// carried this sampler's first two kernels; fold_out: this pass carries the next sampler's.  Folding stays inside one
// graph (the last pass of a graph never folds), so whatever follows a graph starts from a clean histogram.
int enqueue_iteration(sllm_engine* e, const SampleArgs& s, bool fold_in = false, bool fold_out = false) {
    int rc = launch_sampler(e, s, true, fold_in);
    if (rc) return rc;
    return run_pass(e, decode_view(e), nullptr, e->n_live, e->step_logits, true, fold_out ? &s : nullptr);
}

// A graph of `iters` consecutive decode iterations: inside it the head of one iteration and the sampler of the next
// are joined by a programmatic-dependent-launch edge like every other pair of kernels, which a graph boundary is not.
int get_iteration_graph(sllm_engine* e, const SampleArgs& s, int iters, cudaGraphExec_t* out) {
    GraphKey k{};
    k.iters = iters;
    k.n_slots = s.n_slots; k.t = s.temperature; k.p = s.top_p; k.pen = s.penalty; k.eos = s.eos; k.stop = s.stop_token;
    k.seeded = s.seeded; k.stride = s.draws_stride; k.draws = s.draws;
    auto it = e->graphs.find(k);
    if (it != e->graphs.end()) { *out = it->second.first; e->iter_launches = it->second.second; return SLLM_OK; }
    // run once outside capture so that every lazy attribute / module load has happened ...
    // (not needed for correctness of results: capture replays the same launches)
    cudaGraph_t g = nullptr;
    const uint64_t before = e->launches;
    CU(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal));
    int rc = SLLM_OK;
    const bool can_fold = pass_is_persistent(e, e->n_live) && s.n_slots == 1 && e->ps_na <= 128 && e->fold_sampler;   // the pick kernel reads up to 128 parts
    for (int i = 0; i < iters && !rc; ++i) rc = enqueue_iteration(e, s, can_fold && i > 0, can_fold && i + 1 < iters);
    cudaError_t ce = cudaStreamEndCapture(e->stream, &g);
    e->iter_launches = (int)(e->launches - before);
    e->launches = before;
    if (rc) { if (g) cudaGraphDestroy(g); return rc; }
    if (ce != cudaSuccess) return fail(e, SLLM_ERR_CUDA, std::string("graph capture failed: ") + cudaGetErrorString(ce));
    cudaGraphExec_t ge = nullptr;
    ce = cudaGraphInstantiate(&ge, g, 0);
    cudaGraphDestroy(g);
    if (ce != cudaSuccess) return fail(e, SLLM_ERR_CUDA, std::string("graph instantiate failed: ") + cudaGetErrorString(ce));
    if (e->graphs.size() > 32) {
        for (auto& kv : e->graphs) cudaGraphExecDestroy(kv.second.first);
        e->graphs.clear();
    }
    e->graphs[k] = std::make_pair(ge, e->iter_launches);
    *out = ge;
    return SLLM_OK;
}

int launches_per_iteration(const sllm_engine* e) { return e->iter_launches; }

int status_error(sllm_engine* e, unsigned int st) {
    cudaMemsetAsync(e->d_status, 0, sizeof st, e->stream);
    return fail(e, SLLM_ERR_DEVICE_WAIT, "a bounded device-side wait gave up (code " + std::to_string(st) + ")");
}

// Finished flags of the live slots plus the device status word, in one synchronisation.
int check_finished_flags(sllm_engine* e, bool* all_done, bool* nonfinite) {
    int* h_status = e->h_flags + e->max_batch;
    CU(cudaMemcpyAsync(e->h_flags, e->st.finished, e->n_live * sizeof(int), cudaMemcpyDeviceToHost, e->stream));
    CU(cudaMemcpyAsync(h_status, e->d_status, sizeof(int), cudaMemcpyDeviceToHost, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    if (*h_status) return status_error(e, (unsigned int)*h_status);
    *all_done = true; *nonfinite = false;
    for (int s = 0; s < e->n_live; ++s) {
        if (e->h_flags[s] == 0) *all_done = false;
        if (e->h_flags[s] == 3) *nonfinite = true;
    }
    return SLLM_OK;
}

// The draw buffer is allocated once at creation (max_batch x token capacity of a slot): no call of the token loop
// allocates, and the cached graphs keep a valid pointer for the engine's lifetime.
int upload_draws(sllm_engine* e, const double* host, size_t n_slots, size_t stride, bool transpose_from_step_major) {
    const size_t n = n_slots * stride;
    if (n > e->draws_cap)
        return fail(e, SLLM_ERR_CAPACITY, "more draws than the engine's draw buffer holds (max_batch x (2 * context_length + 2)): "
                                          "ask for fewer steps per call");
    if (!transpose_from_step_major || n_slots == 1) {
        CU(cudaMemcpyAsync(e->d_draws, host, n * sizeof(double), cudaMemcpyHostToDevice, e->stream));
        CU(cudaStreamSynchronize(e->stream));
    } else {
        std::vector<double> t(n);
        for (size_t st = 0; st < stride; ++st)
            for (size_t s = 0; s < n_slots; ++s) t[s * stride + st] = host[st * n_slots + s];
        CU(cudaMemcpyAsync(e->d_draws, t.data(), n * sizeof(double), cudaMemcpyHostToDevice, e->stream));
        CU(cudaStreamSynchronize(e->stream));
    }
    return SLLM_OK;
}

// generate_canonical<double,53>(std::mt19937_64): what std::discrete_distribution draws
void canonical_stream(uint64_t seed, size_t n, double* out) {
    std::mt19937_64 g(seed);
    for (size_t i = 0; i < n; ++i) out[i] = std::generate_canonical<double, 53>(g);
}

int find_param(const sllm_engine* e, const char* name) {
    for (size_t i = 0; i < e->params.size(); ++i) if (e->params[i].name == name) return (int)i;
    return -1;
}

template <typename WT>
int convert_param(sllm_engine* e, const ParamSlot& p) {
    const ModelDims& m = e->md;
    const size_t n = p.ndim == 2 ? p.dims[0] * p.dims[1] : p.dims[0];
    auto transpose = [&](void* dst, int K, int N, int mul, int add, int row_off) -> int {
        WT* d = static_cast<WT*>(dst) + (size_t)row_off * K;
        const dim3 grid((N + 31) / 32, (K + 31) / 32), block(32, 8);
        return launch(e, k_repack_transpose<WT>, grid, block, 0, false, (const float*)e->staging, d, K, N, mul, add);
    };
    LayerW* lw = p.layer >= 0 ? &e->layers[p.layer] : nullptr;
    switch (p.kind) {
        case 0: {
            CU(cudaMemcpyAsync(e->emb_f32, e->staging, n * sizeof(float), cudaMemcpyDeviceToDevice, e->stream));
            return launch(e, k_cast<WT>, dim3(e->sm_count * 8), dim3(256), 0, false, (const float*)e->staging,
                          static_cast<WT*>(e->emb_w), n);
        }
        case 1: CU(cudaMemcpyAsync((void*)lw->g_attn, e->staging, n * 4, cudaMemcpyDeviceToDevice, e->stream)); return SLLM_OK;
        case 6: CU(cudaMemcpyAsync((void*)lw->g_ffn, e->staging, n * 4, cudaMemcpyDeviceToDevice, e->stream)); return SLLM_OK;
        case 10: CU(cudaMemcpyAsync(e->g_final, e->staging, n * 4, cudaMemcpyDeviceToDevice, e->stream)); return SLLM_OK;
        case 2: return transpose((void*)lw->wqkv, m.D, m.D, 1, 0, 0);
        case 3: return transpose((void*)lw->wqkv, m.D, m.D, 1, 0, m.D);
        case 4: return transpose((void*)lw->wqkv, m.D, m.D, 1, 0, 2 * m.D);
        case 5: return transpose((void*)lw->wo, m.D, m.D, 1, 0, 0);
        case 7: return transpose((void*)lw->wgu, m.D, m.F, 2, 0, 0);
        case 8: return transpose((void*)lw->wgu, m.D, m.F, 2, 1, 0);
        case 9: {
            int rc = transpose((void*)lw->wd, m.F, m.D, 1, 0, 0);
            if (rc || !e->fused_ok) return rc;
            // the fused decode kernels read the down weights row-per-hidden-unit: the reference's own [F][D]
            return launch(e, k_cast<WT>, dim3(e->sm_count * 4), dim3(256), 0, false, (const float*)e->staging,
                          static_cast<WT*>(e->wdT[p.layer]), n);
        }
    }
    return fail(e, SLLM_ERR_INVALID, "unknown parameter kind");
}

int set_param_impl(sllm_engine* e, int idx, const float* host) {
    const ParamSlot& p = e->params[idx];
    const size_t n = p.ndim == 2 ? p.dims[0] * p.dims[1] : p.dims[0];
    CU(cudaMemcpyAsync(e->staging, host, n * sizeof(float), cudaMemcpyHostToDevice, e->stream));
    int rc = e->f32 ? convert_param<float>(e, p) : convert_param<__nv_bfloat16>(e, p);
    if (rc) return rc;
    CU(cudaStreamSynchronize(e->stream));      // the host buffer may be reused by the caller
    return SLLM_OK;
}

// Teacher-forced loss of one logits row (ops::cross_entropy, src/ops/cross_entropy.cpp:27-50):
// -logit[target] + max + log(sum exp(logit - max)) in fp32; rows with a negative target give 0.
__global__ void __launch_bounds__(256) k_row_loss(const float* __restrict__ logits, const int* __restrict__ targets,
                                                  float* __restrict__ loss, int V) {
    __shared__ float red[8];
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;
    const int tgt = targets[r];
    if (tgt < 0) { if (tid == 0) loss[r] = 0.f; return; }
    const float* l = logits + (size_t)r * V;
    float mx = -INFINITY;
    for (int j = tid; j < V; j += 256) mx = fmaxf(mx, l[j]);
    mx = warp_max(mx);
    if (lane == 0) red[wp] = mx;
    __syncthreads();
    mx = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red[w]);
    __syncthreads();
    float sum = 0.f;
    for (int j = tid; j < V; j += 256) sum += expf(l[j] - mx);
    sum = warp_sum(sum);
    if (lane == 0) red[wp] = sum;
    __syncthreads();
    if (tid == 0) {
        float t = 0.f;
        for (int w = 0; w < 8; ++w) t += red[w];
        loss[r] = -l[tgt] + (mx + logf(t));
    }
}

int load_slots(sllm_engine* e, const uint32_t* ids, const uint32_t* lens, uint32_t n_seq, bool allow_long = false) {
    const ModelDims& m = e->md;
    if (n_seq == 0 || n_seq > (uint32_t)e->max_batch) return fail(e, SLLM_ERR_CAPACITY, "n_seq exceeds max_batch");
    size_t total = 0;
    for (uint32_t s = 0; s < n_seq; ++s) {
        if (lens[s] == 0) return fail(e, SLLM_ERR_INVALID, "Inference::generate: prompt encoded to zero tokens");
        if (lens[s] > (uint32_t)(allow_long ? e->st.tok_cap - 1 : m.ctx))
            return fail(e, SLLM_ERR_INVALID, allow_long ? "prompt longer than the engine's token buffer (2 x context_length)"
                                                        : "Model::forward: seq_len exceeds context_length");
        total += lens[s];
    }
    for (size_t i = 0; i < total; ++i)
        if (ids[i] >= (uint32_t)m.V) return fail(e, SLLM_ERR_INVALID, "token id outside the vocabulary");
    for (int s = 0; s < e->max_batch; ++s) { release_slot(e, s); e->slot_released[s] = 0; }
    e->n_live = (int)n_seq;
    // slot state on the device
    const int cap = e->st.tok_cap, words = m.V / 32;
    std::vector<uint32_t> toks((size_t)n_seq * cap, 0), seen((size_t)n_seq * words, 0);
    std::vector<int> ntok(n_seq), zeros(n_seq, 0), fin(n_seq, 0);
    size_t off = 0;
    for (uint32_t s = 0; s < n_seq; ++s) {
        for (uint32_t i = 0; i < lens[s]; ++i) {
            const uint32_t id = ids[off + i];
            toks[(size_t)s * cap + i] = id;
            seen[(size_t)s * words + (id >> 5)] |= 1u << (id & 31);
        }
        ntok[s] = (int)lens[s];
        off += lens[s];
        bool changed = false;
        e->h_len_bound[s] = std::min<int>((int)lens[s], m.ctx + 1);
        fin[s] = lens[s] > (uint32_t)m.ctx ? 2 : 0;          // window already full: generation starts by sliding
        int rc = ensure_pages(e, (int)s, (int)lens[s], &changed);
        if (rc) return rc;
        rc = upload_block_table(e, (int)s);
        if (rc) return rc;
    }
    CU(cudaMemcpyAsync(e->st.tokens, toks.data(), toks.size() * 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaMemcpyAsync(e->st.seen, seen.data(), seen.size() * 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaMemcpyAsync(e->st.n_tok, ntok.data(), n_seq * 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaMemcpyAsync(e->st.finished, fin.data(), n_seq * 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaMemcpyAsync(e->st.draw_idx, zeros.data(), n_seq * 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    return SLLM_OK;
}

// Final norm + tied head for selected tokens of the pass whose residual stream sits in e->x.
int run_head(sllm_engine* e, const PassView& pv, const int* d_row_tok, int nr, float* out) {
    const ModelDims& m = e->md;
    if (!e->f32 && e->encode_tiled && nr >= e->tc_min_tokens) {
        int rc = launch(e, k_rmsnorm_bf16, dim3(nr), dim3(256), 0, false, (const float*)e->x, (const float*)e->g_final,
                        e->head16, m.D, m.eps, d_row_tok, (const float*)nullptr, pv.tok_id, e->x);
        if (rc) return rc;
        TcArgs h{};
        h.m = m; h.pass = pv; h.status = e->d_status; h.R = m.V; h.K = m.D; h.out = out; h.n_tok = nr;
        return launch_tc<kModeHead>(e, e->map_head, e->head16, e->logit_rows_cap, h, false);
    }
    GemvArgs a{};
    a.m = m; a.eps = m.eps; a.W = e->emb_w; a.R = m.V; a.K = m.D; a.in = e->x; a.gain = e->g_final;
    a.out = out; a.n_tok = nr; a.row_tok = d_row_tok; a.pass = pv;
    return e->f32 ? launch_gemv<float, kModeHead>(e, a, false) : launch_gemv<__nv_bfloat16, kModeHead>(e, a, false);
}

int check_status(sllm_engine* e) {
    unsigned int st = 0;
    CU(cudaMemcpyAsync(&st, e->d_status, sizeof st, cudaMemcpyDeviceToHost, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    if (st) return status_error(e, st);
    return SLLM_OK;
}

// Prompt positions per prefill chunk when the caller leaves the choice to the engine.  A chunk's four projections run
// as 128 x 256 tiles, one block per SM walking its tiles, so a projection takes ceil(tiles / SMs) rounds whatever the
// fill of the last round: 8192 positions of the 100.3M model are 480 / 160 / 864 / 160 tiles = 4 / 2 / 6 / 2 rounds
// on 148 SMs, 7424 positions are 435 / 145 / 783 / 145 tiles = 3 / 1 / 6 / 1 rounds.  Picks the multiple of 256 in
// the upper half of the pass buffers with the fewest modelled microseconds per position (a round costs a tile's time:
// a fixed part for the epilogue -- smaller for the SiLU epilogue, which stores half as much -- plus the K blocks).
int pick_chunk_tokens(int cap, int D, int F, int sms) {
    if (cap < 2048) return cap;
    double best = 0.0; int best_t = cap;
    for (int t = cap - cap % 256; t >= cap / 2; t -= 256) {
        const int tn = (t + 255) / 256;
        auto rounds = [&](int R) { return (double)((((R + kTcBM - 1) / kTcBM) * tn + sms - 1) / sms); };
        const double kd = 0.5 * ((D + kTcBK - 1) / kTcBK), kf = 0.5 * ((F + kTcBK - 1) / kTcBK);
        const double us = rounds(3 * D) * (6.0 + kd) + rounds(D) * (6.0 + kd) + rounds(2 * F) * (2.5 + kd) + rounds(D) * (6.0 + kf);
        const double per_pos = us / t;
        if (best == 0.0 || per_pos < best * 0.995) { best = per_pos; best_t = t; }   // ties go to the larger chunk
    }
    return best_t;
}

// Runs every prompt position through the model in chunks.  want_all: logits of every position go
// to host_logits [sum(lens)][V]; otherwise the last position of each slot goes to step_logits.
// pos0s: first position of each sequence's ids (tokens appended behind what the slot's KV cache already holds).
// h_targets / h_row_loss: instead of logits, every position's teacher-forced loss against its target goes to the host.
int prefill_impl(sllm_engine* e, const uint32_t* ids, const uint32_t* lens, uint32_t n_seq, float* host_logits,
                 const int* slot_ids = nullptr, const int* pos0s = nullptr, const int32_t* h_targets = nullptr,
                 float* h_row_loss = nullptr) {
    const ModelDims& m = e->md;
    std::vector<uint32_t> c_id; std::vector<int> c_slot, c_pos, c_row; std::vector<int> c_row_dst;
    std::vector<PfTile> c_tiles;
    c_id.reserve(e->pass_cap); c_slot.reserve(e->pass_cap); c_pos.reserve(e->pass_cap);
    size_t off = 0, row_base = 0;
    auto flush = [&]() -> int {
        if (c_id.empty()) return SLLM_OK;
        const int n = (int)c_id.size();
        // the attention grid takes its tiles in this order: the ones with the most KV pages first, so that the last
        // wave of blocks is the shortest
        std::stable_sort(c_tiles.begin(), c_tiles.end(),
                         [](const PfTile& x, const PfTile& y) { return x.pos0 + x.n_q > y.pos0 + y.n_q; });
        // this chunk's lists go through one of two pinned buffers: [ids | slots | positions | row list | tiles]
        const int b = e->pf_next;
        e->pf_next ^= 1;
        if (e->ev_pf_used[b]) CU(cudaEventSynchronize(e->ev_pf[b]));       // its previous contents have been copied
        unsigned char* hp = e->h_pf[b];
        uint32_t* h_id = reinterpret_cast<uint32_t*>(hp);
        int* h_slot = reinterpret_cast<int*>(hp) + e->pass_cap;
        int* h_pos = h_slot + e->pass_cap;
        int* h_row = h_pos + e->pass_cap;
        PfTile* h_tiles = reinterpret_cast<PfTile*>(h_row + e->pass_cap);
        std::memcpy(h_id, c_id.data(), (size_t)n * 4);
        std::memcpy(h_slot, c_slot.data(), (size_t)n * 4);
        std::memcpy(h_pos, c_pos.data(), (size_t)n * 4);
        std::memcpy(h_row, c_row.data(), c_row.size() * 4);
        std::memcpy(h_tiles, c_tiles.data(), c_tiles.size() * sizeof(PfTile));
        CU(cudaMemcpyAsync(e->d_tok_id, h_id, (size_t)n * 4, cudaMemcpyHostToDevice, e->stream));
        CU(cudaMemcpyAsync(e->d_tok_slot, h_slot, (size_t)n * 4, cudaMemcpyHostToDevice, e->stream));
        CU(cudaMemcpyAsync(e->d_tok_pos, h_pos, (size_t)n * 4, cudaMemcpyHostToDevice, e->stream));
        CU(cudaMemcpyAsync(e->d_tiles, h_tiles, c_tiles.size() * sizeof(PfTile), cudaMemcpyHostToDevice, e->stream));
        PassView pv{e->d_tok_id, e->d_tok_slot, e->d_tok_pos, n, e->d_tiles, (int)c_tiles.size()};
        e->prefill_tokens += (uint64_t)n;
        int rc = run_pass(e, pv, nullptr, 0, nullptr, false);
        if (rc) return rc;
        // logits rows of this chunk, in groups that fit the logits buffer
        for (size_t r0 = 0; r0 < c_row.size(); r0 += e->logit_rows_cap) {
            const int nr = (int)std::min<size_t>(e->logit_rows_cap, c_row.size() - r0);
            CU(cudaMemcpyAsync(e->d_row_tok, h_row + r0, nr * 4, cudaMemcpyHostToDevice, e->stream));
            rc = run_head(e, pv, e->d_row_tok, nr, e->pass_logits);
            if (rc) return rc;
            if (h_targets) {
                CU(cudaMemcpyAsync(e->d_row_target, h_targets + row_base + r0, (size_t)nr * 4, cudaMemcpyHostToDevice, e->stream));
                k_row_loss<<<nr, 256, 0, e->stream>>>(e->pass_logits, e->d_row_target, e->d_row_loss, m.V);
                CU(cudaGetLastError());
                e->launches += 1;
                CU(cudaMemcpyAsync(h_row_loss + row_base + r0, e->d_row_loss, (size_t)nr * 4, cudaMemcpyDeviceToHost, e->stream));
            } else if (host_logits) {
                CU(cudaMemcpyAsync(host_logits + (row_base + r0) * m.V, e->pass_logits, (size_t)nr * m.V * 4,
                                   cudaMemcpyDeviceToHost, e->stream));
            } else {
                for (int i = 0; i < nr; ++i)
                    CU(cudaMemcpyAsync(e->step_logits + (size_t)c_row_dst[r0 + i] * m.V, e->pass_logits + (size_t)i * m.V,
                                       (size_t)m.V * 4, cudaMemcpyDeviceToDevice, e->stream));
            }
            // results for the host: the caller's buffers and the target list are reused per group
            if (h_targets || host_logits) CU(cudaStreamSynchronize(e->stream));
        }
        CU(cudaEventRecord(e->ev_pf[b], e->stream));             // every copy out of this staging buffer is enqueued before here
        e->ev_pf_used[b] = true;
        row_base += c_row.size();
        c_id.clear(); c_slot.clear(); c_pos.clear(); c_row.clear(); c_row_dst.clear(); c_tiles.clear();
        return SLLM_OK;
    };
    for (uint32_t s = 0; s < n_seq; ++s) {
        for (uint32_t i = 0; i < lens[s]; ++i) {
            if ((int)c_id.size() == e->chunk_tokens) { int rc = flush(); if (rc) return rc; }
            const int slot = slot_ids ? slot_ids[s] : (int)s;
            const int pos = (pos0s ? pos0s[s] : 0) + (int)i;
            if (host_logits || h_targets || i + 1 == lens[s]) { c_row.push_back((int)c_id.size()); c_row_dst.push_back(slot); }
            if (!c_tiles.empty() && c_tiles.back().slot == slot && c_tiles.back().n_q < e->pf_tile_q &&
                c_tiles.back().pos0 + c_tiles.back().n_q == pos && c_tiles.back().tok_begin + c_tiles.back().n_q == (int)c_id.size())
                c_tiles.back().n_q += 1;
            else
                c_tiles.push_back(PfTile{(int)c_id.size(), 1, slot, pos});
            c_id.push_back(ids[off + i]); c_slot.push_back(slot); c_pos.push_back(pos);
        }
        off += lens[s];
    }
    int rc = flush();
    if (rc) return rc;
    return check_status(e);
}

}  // namespace

// =================================================================================== C ABI ===
extern "C" {

void sllm_default_model_config(sllm_model_config* c) {
    c->vocab_size = 32768; c->context_length = 2048; c->num_layers = 16; c->d_model = 640;
    c->num_heads = 10; c->ffn_hidden = 1728; c->rope_theta = 10000.0f; c->rms_eps = 1e-5f;
}
void sllm_default_engine_options(sllm_engine_options* o) {
    std::memset(o, 0, sizeof *o);
    o->max_batch = 1; o->weight_dtype = SLLM_WEIGHTS_BF16; o->kv_pages = 0; o->max_chunk_tokens = 0;
    o->device = -1; o->use_graph = 1;
}
void sllm_default_sampling(sllm_sampling* s) {
    s->temperature = 0.7f; s->top_p = 0.8f; s->repetition_penalty = 1.1f; s->eos_token = 32762;
    s->stop_token = -1; s->seed = 1234;
}

const char* sllm_last_error(const sllm_engine* e) { return e ? e->err.c_str() : g_create_error.c_str(); }

int sllm_engine_create(const sllm_model_config* cfg, const sllm_engine_options* opt_in, sllm_engine** out) {
    if (!cfg || !out) return fail(nullptr, SLLM_ERR_INVALID, "sllm_engine_create: null argument");
    *out = nullptr;
    sllm_engine_options opt;
    if (opt_in) opt = *opt_in; else sllm_default_engine_options(&opt);
    const uint64_t V = cfg->vocab_size, D = cfg->d_model, H = cfg->num_heads, F = cfg->ffn_hidden, L = cfg->num_layers;
    if (!V || !D || !H || !F || !L) return fail(nullptr, SLLM_ERR_INVALID, "model config has a zero dimension");
    if (cfg->context_length == 0)
        return fail(nullptr, SLLM_ERR_INVALID, "Inference::generate: context length must be greater than zero");
    if (D % H) return fail(nullptr, SLLM_ERR_INVALID, "Attention: d_model must equal num_heads * head_dim");
    const uint64_t hd = D / H;
    if (hd != 16 && hd != 32 && hd != 64 && hd != 128) return fail(nullptr, SLLM_ERR_INVALID, "head_dim must be 16, 32, 64 or 128");
    if (D % 8 || F % 8 || V % 64) return fail(nullptr, SLLM_ERR_INVALID, "d_model and ffn_hidden must be multiples of 8, vocab_size of 64");
    if (V > 49152) return fail(nullptr, SLLM_ERR_INVALID, "vocab_size above 49152 does not fit the sampler's shared memory");
    if (opt.max_batch == 0) return fail(nullptr, SLLM_ERR_INVALID, "max_batch must be at least 1");

    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
        cudaGetLastError();
        return fail(nullptr, SLLM_ERR_CUDA, "no CUDA device: this library has no CPU path");
    }
    sllm_engine* e = new sllm_engine();
    e->cfg = *cfg; e->opt = opt; e->f32 = opt.weight_dtype == SLLM_WEIGHTS_F32;
    auto bail = [&](int rc) { g_create_error = e->err; sllm_engine_destroy(e); return rc; };
    if (opt.device >= 0) { if (cudaSetDevice(opt.device) != cudaSuccess) { e->err = "cudaSetDevice failed"; return bail(SLLM_ERR_CUDA); } }
    cudaGetDevice(&e->dev);
    cudaDeviceProp prop{};
    if (cudaGetDeviceProperties(&prop, e->dev) != cudaSuccess) { e->err = "cudaGetDeviceProperties failed"; return bail(SLLM_ERR_CUDA); }
    if (prop.major != 10) {
        e->err = "device compute capability " + std::to_string(prop.major) + "." + std::to_string(prop.minor) +
                 " is not 10.x: the kernels are built for sm_100a only";
        return bail(SLLM_ERR_CUDA);
    }
    e->sm_count = prop.multiProcessorCount;
    e->max_dyn_smem = prop.sharedMemPerBlockOptin;
    if (cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking) != cudaSuccess) { e->err = "cudaStreamCreate failed"; return bail(SLLM_ERR_CUDA); }
    cudaEventCreate(&e->ev0); cudaEventCreate(&e->ev1);

    ModelDims& m = e->md;
    m.V = (int)V; m.ctx = (int)cfg->context_length; m.L = (int)L; m.D = (int)D; m.H = (int)H; m.hd = (int)hd; m.F = (int)F;
    m.eps = cfg->rms_eps; m.scale = 1.0f / std::sqrt((float)hd);
    e->max_batch = (int)opt.max_batch;
    e->pages_per_seq = (m.ctx + kPage - 1) / kPage;
    e->n_pages = (opt.kv_pages ? (long long)opt.kv_pages : (long long)e->max_batch * e->pages_per_seq) + 1;   // + the spare page
    e->spare_page = (int)(e->n_pages - 1);
    if (const char* v = std::getenv("SLLM_WAIT_LIMIT_MS")) {        // diagnostic: how long a device-side wait polls before it gives up
        const unsigned long long ns = (unsigned long long)std::min(std::max(std::atoll(v), 1ll), 60000ll) * 1000000ull;
        if (cudaMemcpyToSymbol(c_wait_limit_ns, &ns, sizeof ns) != cudaSuccess) { e->err = "cannot set the wait limit"; return bail(SLLM_ERR_CUDA); }
    }
    if (const char* v = std::getenv("SLLM_TC_MIN_TOKENS")) e->tc_min_tokens = std::max(1, std::atoi(v));   // tuning aid
    if (const char* v = std::getenv("SLLM_TC_SPLIT")) e->tune_tc_split = std::max(0, std::atoi(v));
    if (std::getenv("SLLM_NO_PERSISTENT_TC")) e->tune_no_persistent_tc = 1;
    if (std::getenv("SLLM_NO_WIDE_EPI")) e->tune_no_wide_epi = 1;
    if (const char* v = std::getenv("SLLM_ORDER_WAVES")) e->order_min_waves = std::max(1, std::atoi(v));
    if (const char* v = std::getenv("SLLM_STREAM_SPLITS")) e->tune_stream_splits = std::min(std::max(0, std::atoi(v)), 8);
    e->pass_cap = opt.max_chunk_tokens ? (int)opt.max_chunk_tokens : 8192;
    e->pass_cap = std::max(e->pass_cap, e->max_batch);
    e->chunk_tokens = e->pass_cap;
    if (!opt.max_chunk_tokens && !e->f32) e->chunk_tokens = std::max(e->max_batch, pick_chunk_tokens(e->pass_cap, (int)D, (int)F, e->sm_count));
    if (const char* v = std::getenv("SLLM_CHUNK_TOKENS")) e->chunk_tokens = std::min(e->pass_cap, std::max(e->max_batch, std::atoi(v)));
    e->logit_rows_cap = std::max(e->max_batch, 64);

    // registry: src/model.cpp:106-131
    auto add = [&](const std::string& n, uint64_t d0, uint64_t d1, int kind, int layer) {
        ParamSlot p; p.name = n; p.dims[0] = d0; p.dims[1] = d1; p.ndim = d1 ? 2 : 1; p.kind = kind; p.layer = layer;
        e->params.push_back(p);
    };
    add("embedding", V, D, 0, -1);
    for (uint64_t l = 0; l < L; ++l) {
        const std::string pre = "blocks." + std::to_string(l) + ".";
        add(pre + "attn_norm", D, 0, 1, (int)l);
        add(pre + "attn.q", D, D, 2, (int)l); add(pre + "attn.k", D, D, 3, (int)l);
        add(pre + "attn.v", D, D, 4, (int)l); add(pre + "attn.out", D, D, 5, (int)l);
        add(pre + "ffn_norm", D, 0, 6, (int)l);
        add(pre + "ffn.gate", D, F, 7, (int)l); add(pre + "ffn.up", D, F, 8, (int)l); add(pre + "ffn.down", F, D, 9, (int)l);
    }
    add("final_norm", D, 0, 10, -1);

    int rc = SLLM_OK;
    const size_t ws = wsize(e);
    auto A = [&](auto** p, size_t n, uint64_t* ctr) { if (!rc) rc = dalloc(e, p, n, ctr); };
    // weights
    unsigned char* tmp = nullptr;
    A(&tmp, V * D * ws, &e->weight_bytes); e->emb_w = tmp;
    A(&e->emb_f32, V * D, &e->weight_bytes);
    A(&e->g_final, D, &e->weight_bytes);
    e->layers.resize(L);
    std::vector<float> ones(D, 1.0f);
    for (uint64_t l = 0; l < L && !rc; ++l) {
        LayerW& w = e->layers[l];
        unsigned char* p = nullptr; float* g = nullptr;
        A(&p, 3 * D * D * ws, &e->weight_bytes); w.wqkv = p;
        A(&p, D * D * ws, &e->weight_bytes); w.wo = p;
        A(&p, 2 * F * D * ws, &e->weight_bytes); w.wgu = p;
        A(&p, D * F * ws, &e->weight_bytes); w.wd = p;
        A(&g, D, &e->weight_bytes); w.g_attn = g;
        A(&g, D, &e->weight_bytes); w.g_ffn = g;
        if (!rc) {
            cudaMemcpyAsync((void*)w.g_attn, ones.data(), D * 4, cudaMemcpyHostToDevice, e->stream);
            cudaMemcpyAsync((void*)w.g_ffn, ones.data(), D * 4, cudaMemcpyHostToDevice, e->stream);
        }
    }
    if (!rc) cudaMemcpyAsync(e->g_final, ones.data(), D * 4, cudaMemcpyHostToDevice, e->stream);
    e->staging_elems = std::max<size_t>({V * D, D * F, D * D});
    A(&e->staging, e->staging_elems, &e->scratch_bytes);
    // RoPE table with the reference's fp32 expressions, src/ops/rope.cpp:48-56
    {
        std::vector<float2> tab((size_t)m.ctx * (hd / 2));
        for (int pos = 0; pos < m.ctx; ++pos)
            for (uint64_t i = 0; i < hd / 2; ++i) {
                const float frequency = 1.0f / std::pow(cfg->rope_theta, static_cast<float>(2 * i) / static_cast<float>(hd));
                const float angle = static_cast<float>(pos) * frequency;
                tab[(size_t)pos * (hd / 2) + i] = make_float2(std::cos(angle), std::sin(angle));
            }
        A(&e->rope, tab.size(), &e->weight_bytes);
        if (!rc) cudaMemcpyAsync(e->rope, tab.data(), tab.size() * sizeof(float2), cudaMemcpyHostToDevice, e->stream);
        if (!rc) cudaStreamSynchronize(e->stream);
    }
    // KV pool
    {
        unsigned char* p = nullptr;
        const size_t page_bytes = 2 * H * kPage * hd * ws;
        if (!rc) {
            void* q = nullptr;
            const size_t bytes = (size_t)L * e->n_pages * page_bytes;
            cudaError_t ce = cudaMalloc(&q, bytes);
            if (ce != cudaSuccess) { e->err = std::string("KV pool allocation failed: ") + cudaGetErrorString(ce); rc = SLLM_ERR_CUDA; }
            else {
                e->allocs.push_back(q); e->kv_pool = q; e->kv_bytes = bytes;
                // Kernels that multiply whole pages by zero probabilities (the tensor-core prefill attention) need
                // finite values in rows no position has written yet: 0 x Inf/NaN would poison the product.  Pages
                // that return to the pool hold finite K/V of their previous owner, so clearing once suffices.
                cudaMemsetAsync(q, 0, bytes, e->stream);
            }
        }
        (void)p;
        e->free_pages.resize(e->n_pages - 1);
        for (long long i = 0; i + 1 < e->n_pages; ++i) e->free_pages[i] = (int)(e->n_pages - 2 - i);
        e->slot_pages.assign(e->max_batch, {});
        e->slot_released.assign(e->max_batch, 0);
        e->h_len_bound.assign(e->max_batch, 0);
        A(&e->d_block_table, (size_t)e->max_batch * e->pages_per_seq, &e->scratch_bytes);
    }
    // slot state
    e->st.tok_cap = 2 * m.ctx + 2;     // room for the window to slide by one context length
    A(&e->st.tokens, (size_t)e->max_batch * e->st.tok_cap, &e->scratch_bytes);
    A(&e->st.n_tok, e->max_batch, &e->scratch_bytes);
    A(&e->st.finished, e->max_batch, &e->scratch_bytes);
    A(&e->st.seen, (size_t)e->max_batch * (V / 32), &e->scratch_bytes);
    A(&e->st.draw_idx, e->max_batch, &e->scratch_bytes);
    // pass buffers
    A(&e->d_tok_id, e->pass_cap, &e->scratch_bytes); A(&e->d_tok_slot, e->pass_cap, &e->scratch_bytes);
    A(&e->d_tok_pos, e->pass_cap, &e->scratch_bytes);
    A(&e->d_dec_id, e->max_batch, &e->scratch_bytes); A(&e->d_dec_slot, e->max_batch, &e->scratch_bytes);
    A(&e->d_attn_order, e->max_batch, &e->scratch_bytes);
    A(&e->d_dec_pos, e->max_batch, &e->scratch_bytes);
    A(&e->d_row_tok, e->pass_cap, &e->scratch_bytes);
    A(&e->d_row_target, e->logit_rows_cap, &e->scratch_bytes); A(&e->d_row_loss, e->logit_rows_cap, &e->scratch_bytes);
    A(&e->d_tiles, e->pass_cap, &e->scratch_bytes);
    A(&e->x, (size_t)e->pass_cap * D, &e->scratch_bytes); A(&e->q, (size_t)e->pass_cap * D, &e->scratch_bytes);
    A(&e->att, (size_t)e->pass_cap * D, &e->scratch_bytes); A(&e->hid, (size_t)e->pass_cap * F, &e->scratch_bytes);
    A(&e->step_logits, (size_t)e->max_batch * V, &e->scratch_bytes);
    A(&e->pass_logits, (size_t)e->logit_rows_cap * V, &e->scratch_bytes);
    {   // fused single-token path: shapes it supports
        const int epc = e->f32 ? 4 : 8;
        const int nch = (int)D / epc;
        e->fused_upc = std::max<int>((int)((F + 143) / 144), 2);
        e->fused_nb = (int)(((F + e->fused_upc - 1) / e->fused_upc + kCS - 1) / kCS) * kCS;
        e->fused_ok = nch <= kFusedThreads && e->fused_upc <= 64 && D % kCS == 0 &&
                      (size_t)(2 + std::max(kFusedThreads / nch, 2)) * D * sizeof(float) <= 48 * 1024;
        if (e->fused_ok) {
            A(&e->xb, D, &e->scratch_bytes);
            A(&e->attn_parts, H * D, &e->scratch_bytes);
            A(&e->down_parts, (size_t)(e->fused_nb / kCS) * D, &e->scratch_bytes);
            e->wdT.resize(L);
            for (uint64_t l = 0; l < L; ++l) { unsigned char* p = nullptr; A(&p, D * F * ws, &e->weight_bytes); e->wdT[l] = p; }
        }
    }
    A(&e->samp_mass, (size_t)e->max_batch * kL0Buckets, &e->scratch_bytes);
    A(&e->samp_cnt, (size_t)e->max_batch * kL0Buckets, &e->scratch_bytes);
    A(&e->samp_w, (size_t)e->max_batch * V, &e->scratch_bytes);
    A(&e->samp_pmax_val, (size_t)e->max_batch * e->samp_bps_cap, &e->scratch_bytes);
    A(&e->samp_pmax_idx, (size_t)e->max_batch * e->samp_bps_cap, &e->scratch_bytes);
    A(&e->d_status, 4, &e->scratch_bytes);
    e->draws_cap = (size_t)e->max_batch * (size_t)e->st.tok_cap;
    A(&e->d_draws, e->draws_cap, &e->scratch_bytes);
    if (!e->f32) {
        A(&e->xn16, (size_t)e->pass_cap * D, &e->scratch_bytes); A(&e->att16, (size_t)e->pass_cap * D, &e->scratch_bytes);
        e->ss_parts = 4 * (int)((D + kTcBM - 1) / kTcBM);
        A(&e->ss_part, (size_t)e->pass_cap * e->ss_parts, &e->scratch_bytes);
        A(&e->hid16, (size_t)e->pass_cap * F, &e->scratch_bytes); A(&e->head16, (size_t)e->logit_rows_cap * D, &e->scratch_bytes);
        cudaDriverEntryPointQueryResult qres;
        if (!rc && (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &e->encode_tiled, cudaEnableDefault, &qres) != cudaSuccess ||
                    qres != cudaDriverEntryPointSuccess || !e->encode_tiled)) {
            e->err = "cuTensorMapEncodeTiled is not available from this driver"; rc = SLLM_ERR_CUDA;
        }
        e->map_wqkv.resize(L); e->map_wo.resize(L); e->map_wgu.resize(L); e->map_wd.resize(L);
        for (uint64_t l = 0; l < L && !rc; ++l) {
            rc = make_map(e, &e->map_wqkv[l], e->layers[l].wqkv, 3 * D, D, kTcBM);
            if (!rc) rc = make_map(e, &e->map_wo[l], e->layers[l].wo, D, D, kTcBM);
            if (!rc) rc = make_map(e, &e->map_wgu[l], e->layers[l].wgu, 2 * F, D, kTcBM);
            if (!rc) rc = make_map(e, &e->map_wd[l], e->layers[l].wd, D, F, kTcBM);
        }
        if (!rc) rc = make_map(e, &e->map_head, e->emb_w, V, D, kTcBM);
        // tensor-core prefill attention: head_dim 64, the pool as one [rows][64] tensor whose rows fit a TMA coordinate
        const unsigned long long kv_rows = (unsigned long long)L * (unsigned long long)e->n_pages * 2ull * H * kPage;
        if (!rc && kv_rows >= (1ull << 32)) {      // the projection epilogue addresses KV rows with 32-bit indices
            e->err = "KV pool has more than 2^32 rows of head_dim elements"; rc = SLLM_ERR_CAPACITY;
        }
        if (!rc && hd == 64 && kv_rows < (1ull << 31) && std::getenv("SLLM_NO_ATTN_TC") == nullptr) {
            rc = make_map(e, &e->map_kv, e->kv_pool, kv_rows, 64, kPage);
            if (!rc && cudaFuncSetAttribute(k_attn_prefill_tc, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            (int)attn_prefill_tc_smem()) != cudaSuccess) {
                e->err = "cudaFuncSetAttribute failed for the prefill attention kernel"; rc = SLLM_ERR_CUDA;
            }
            if (!rc) { e->attn_tc = true; e->pf_tile_q = kPtQ; }
        }
        // persistent single-token decode: every block of the grid must own rows of every product, and its slices fit
        if (!rc && std::getenv("SLLM_NO_PERSIST") == nullptr) {
            // Not every SM: measured on a 148-SM part, 124-132 blocks give 257-260 us per token against 272-275 us with
            // 136-148 (and 290 us with 104): the sampler kernels between two tokens, and the next token's blocks that
            // start early, find free SMs instead of queueing behind blocks that hold all of an SM's shared memory.
            int nc = e->sm_count > 40 ? e->sm_count - 20 : e->sm_count;
            e->fold_sampler = std::getenv("SLLM_NO_FOLD") == nullptr;
            if (const char* v = std::getenv("SLLM_PERSIST_CTAS")) nc = std::max(1, std::min(nc, std::atoi(v)));
            const int na = (int)std::min<uint64_t>({(uint64_t)nc, D, F, 3 * D / 2});
            if (na >= (int)H && L <= 120) {
                const int s_max = na / (int)H;
                const int pps_max = std::max(2, (e->pages_per_seq + s_max - 1) / s_max);
                // the launch takes all the shared memory an SM offers: what the layers leave free holds early head stages
                const PsLayout lay = ps_layout(m, na, s_max, pps_max, e->pages_per_seq, (uint32_t)e->max_dyn_smem);
                if (lay.total <= e->max_dyn_smem && lay.head_stages + lay.head_pre >= 2 && pps_max <= 8) {
                    e->ps_na = na; e->ps_smax = s_max; e->ps_ppsmax = pps_max; e->ps_smem = e->max_dyn_smem;
                    A(&e->ps_xa, D, &e->scratch_bytes); A(&e->ps_xb, D, &e->scratch_bytes);
                    A(&e->ps_qkv, 3 * D, &e->scratch_bytes);
                    A(&e->ps_ap, (size_t)H * s_max * (hd + 2), &e->scratch_bytes);
                    A(&e->ps_hb, F, &e->scratch_bytes);
                    A(&e->ps_epoch, 4, &e->scratch_bytes);
                    A(&e->ps_mxb, 2 * (size_t)na, &e->scratch_bytes);
                    A(&e->d_layers, L, &e->scratch_bytes);
                    if (!rc) {
                        const unsigned int one = 1;
                        cudaMemcpyAsync(e->ps_epoch, &one, sizeof one, cudaMemcpyHostToDevice, e->stream);
                        cudaMemcpyAsync(e->d_layers, e->layers.data(), L * sizeof(LayerW), cudaMemcpyHostToDevice, e->stream);
                        cudaStreamSynchronize(e->stream);
                        cudaError_t ce = cudaSuccess;
                        switch (hd) {
                            case 16: ce = cudaFuncSetAttribute(k_decode_persist<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)e->ps_smem); break;
                            case 32: ce = cudaFuncSetAttribute(k_decode_persist<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)e->ps_smem); break;
                            case 64: ce = cudaFuncSetAttribute(k_decode_persist<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)e->ps_smem); break;
                            default: ce = cudaFuncSetAttribute(k_decode_persist<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)e->ps_smem); break;
                        }
                        if (ce != cudaSuccess) { e->err = "cudaFuncSetAttribute failed for the persistent decode kernel"; rc = SLLM_ERR_CUDA; }
                        else e->persist_ok = true;
                    }
                }
            }
        }
        if (!rc) rc = configure_tc<kModeQKV>(e);
        if (!rc) rc = configure_tc<kModeResidual>(e);
        if (!rc) rc = configure_tc<kModeGateUp>(e);
        if (!rc) rc = configure_tc<kModeHead>(e);
    }
    A(&e->part_o, (size_t)e->split_tok_cap * H * kMaxSplits * hd, &e->scratch_bytes);
    A(&e->part_ml, (size_t)e->split_tok_cap * H * kMaxSplits * 2, &e->scratch_bytes);
    A(&e->ticket, (size_t)e->split_tok_cap * H, &e->scratch_bytes);
    for (int b = 0; b < 2 && !rc; ++b) {
        if (cudaMallocHost((void**)&e->h_pf[b], (size_t)e->pass_cap * (4 * sizeof(int) + sizeof(PfTile))) != cudaSuccess ||
            cudaEventCreateWithFlags(&e->ev_pf[b], cudaEventDisableTiming) != cudaSuccess) {
            e->err = "cudaMallocHost failed"; rc = SLLM_ERR_CUDA;
        }
    }
    if (!rc && cudaMallocHost((void**)&e->h_flags, (e->max_batch + 16) * sizeof(int)) != cudaSuccess) {
        e->err = "cudaMallocHost failed"; rc = SLLM_ERR_CUDA;
    }
    if (!rc && cudaStreamSynchronize(e->stream) != cudaSuccess) { e->err = "initialisation failed"; rc = SLLM_ERR_CUDA; }
    if (!rc) rc = configure_kernels(e);
    if (rc) return bail(rc);
    *out = e;
    return SLLM_OK;
}

void sllm_engine_destroy(sllm_engine* e) {
    if (!e) return;
    if (e->stream) cudaStreamSynchronize(e->stream);
    for (auto& kv : e->graphs) cudaGraphExecDestroy(kv.second.first);
    for (void* p : e->allocs) cudaFree(p);
    if (e->h_flags) cudaFreeHost(e->h_flags);
    for (int b = 0; b < 2; ++b) { if (e->h_pf[b]) cudaFreeHost(e->h_pf[b]); if (e->ev_pf[b]) cudaEventDestroy(e->ev_pf[b]); }
    for (cudaEvent_t ev : e->step_events) cudaEventDestroy(ev);
    if (e->ev0) cudaEventDestroy(e->ev0);
    if (e->ev1) cudaEventDestroy(e->ev1);
    if (e->stream) cudaStreamDestroy(e->stream);
    delete e;
}

int sllm_engine_stats(sllm_engine* e, sllm_stats* s) {
    if (!e || !s) return SLLM_ERR_INVALID;
    s->weight_bytes = e->weight_bytes; s->kv_bytes = e->kv_bytes; s->scratch_bytes = e->scratch_bytes;
    s->kv_pages_total = (uint64_t)e->n_pages - 1; s->kv_pages_free = e->free_pages.size();
    s->launches = e->launches; s->decode_steps = e->decode_steps; s->last_step_ms = e->last_step_ms;
    s->reserved = 0; s->prefill_tokens = e->prefill_tokens;
    return SLLM_OK;
}

void* sllm_engine_stream(sllm_engine* e) { return e ? (void*)e->stream : nullptr; }

uint32_t sllm_num_params(const sllm_engine* e) { return e ? (uint32_t)e->params.size() : 0; }

int sllm_param_info(const sllm_engine* e, uint32_t i, char name[64], uint64_t dims[2], uint32_t* ndim) {
    if (!e || i >= e->params.size()) return SLLM_ERR_INVALID;
    const ParamSlot& p = e->params[i];
    if (name) std::snprintf(name, 64, "%s", p.name.c_str());
    if (dims) { dims[0] = p.dims[0]; dims[1] = p.dims[1]; }
    if (ndim) *ndim = p.ndim;
    return SLLM_OK;
}

int sllm_set_param(sllm_engine* e, const char* name, const float* host, const uint64_t* dims, uint32_t ndim) {
    if (!e || !name || !host || !dims) return fail(e, SLLM_ERR_INVALID, "sllm_set_param: null argument");
    const int idx = find_param(e, name);
    if (idx < 0) return fail(e, SLLM_ERR_INVALID, std::string("unknown parameter '") + name + "'");
    const ParamSlot& p = e->params[idx];
    if (ndim != p.ndim || dims[0] != p.dims[0] || (ndim == 2 && dims[1] != p.dims[1]))
        return fail(e, SLLM_ERR_INVALID, "load_checkpoint: shape mismatch for '" + p.name + "'");
    return set_param_impl(e, idx, host);
}

int sllm_load_checkpoint(sllm_engine* e, const char* path, uint64_t* step, uint64_t* data_position) {
    if (!e || !path) return fail(e, SLLM_ERR_INVALID, "sllm_load_checkpoint: null argument");
    FILE* f = std::fopen(path, "rb");
    if (!f) return fail(e, SLLM_ERR_IO, std::string("load_checkpoint: cannot open ") + path);
    uint64_t st = 0, dp = 0; uint32_t np = 0;
    std::vector<float> host(e->staging_elems);
    auto done = [&](int rc, const std::string& msg) { std::fclose(f); return fail(e, rc, msg); };
    bool ok = std::fread(&st, 8, 1, f) == 1 && std::fread(&dp, 8, 1, f) == 1 && std::fread(&np, 4, 1, f) == 1;
    if (ok && np != e->params.size()) return done(SLLM_ERR_IO, "load_checkpoint: parameter count differs (different model config?)");
    for (size_t i = 0; ok && i < e->params.size(); ++i) {
        const ParamSlot& p = e->params[i];
        uint32_t nl = 0, nd = 0;
        std::string name;
        if (std::fread(&nl, 4, 1, f) == 1 && nl < 4096) { name.resize(nl); if (nl && std::fread(&name[0], 1, nl, f) != nl) name.clear(); }
        if (name != p.name) return done(SLLM_ERR_IO, "load_checkpoint: expected parameter '" + p.name + "', file has '" + name + "'");
        uint64_t dims[4] = {0, 0, 0, 0};
        ok = std::fread(&nd, 4, 1, f) == 1 && nd <= 4;
        for (uint32_t d = 0; ok && d < nd; ++d) ok = std::fread(&dims[d], 8, 1, f) == 1;
        if (!ok) break;
        if (nd != p.ndim || dims[0] != p.dims[0] || (nd == 2 && dims[1] != p.dims[1]))
            return done(SLLM_ERR_IO, "load_checkpoint: shape mismatch for '" + p.name + "'");
        const size_t n = p.ndim == 2 ? p.dims[0] * p.dims[1] : p.dims[0];
        ok = std::fread(host.data(), sizeof(float), n, f) == n;
        if (!ok) break;
        int rc = set_param_impl(e, (int)i, host.data());
        if (rc) { std::fclose(f); return rc; }
    }
    if (!ok) return done(SLLM_ERR_IO, "load_checkpoint: file truncated or corrupt");
    std::fclose(f);
    if (step) *step = st;
    if (data_position) *data_position = dp;
    return SLLM_OK;
}

int sllm_reset(sllm_engine* e) {
    if (!e) return SLLM_ERR_INVALID;
    for (int s = 0; s < e->max_batch; ++s) release_slot(e, s);
    e->n_live = 0;
    return SLLM_OK;
}

int sllm_prefill(sllm_engine* e, const uint32_t* ids, const uint32_t* lens, uint32_t n_seq) {
    if (!e || !ids || !lens) return fail(e, SLLM_ERR_INVALID, "sllm_prefill: null argument");
    int rc = load_slots(e, ids, lens, n_seq);
    if (rc) return rc;
    return prefill_impl(e, ids, lens, n_seq, nullptr);
}

int sllm_forward_logits(sllm_engine* e, const uint32_t* ids, uint64_t B, uint64_t T, float* host_logits) {
    if (!e || !ids || !host_logits) return fail(e, SLLM_ERR_INVALID, "sllm_forward_logits: null argument");
    if (T > (uint64_t)e->md.ctx) return fail(e, SLLM_ERR_INVALID, "Model::forward: seq_len exceeds context_length");
    if (B == 0 || T == 0) return SLLM_OK;
    // rows beyond max_batch are processed in groups of max_batch sequences
    for (uint64_t b0 = 0; b0 < B; b0 += e->max_batch) {
        const uint32_t nb = (uint32_t)std::min<uint64_t>(e->max_batch, B - b0);
        std::vector<uint32_t> lens(nb, (uint32_t)T);
        int rc = load_slots(e, ids + b0 * T, lens.data(), nb);
        if (rc) return rc;
        rc = prefill_impl(e, ids + b0 * T, lens.data(), nb, host_logits + b0 * T * e->md.V);
        if (rc) return rc;
    }
    return SLLM_OK;
}

int sllm_eval_loss(sllm_engine* e, const uint32_t* ids, const int32_t* targets, uint64_t B, uint64_t T, uint64_t num_valid,
                   float* loss) {
    if (!e || !ids || !targets || !loss) return fail(e, SLLM_ERR_INVALID, "sllm_eval_loss: null argument");
    if (B == 0 || T == 0) return fail(e, SLLM_ERR_INVALID, "sllm_eval_loss: empty batch");
    if (T > (uint64_t)e->md.ctx) return fail(e, SLLM_ERR_INVALID, "Model::forward: seq_len exceeds context_length");
    for (uint64_t i = 0; i < B * T; ++i)
        if (targets[i] >= e->md.V) return fail(e, SLLM_ERR_INVALID, "sllm_eval_loss: target outside the vocabulary");
    std::vector<float> row_loss(B * T, 0.f);
    for (uint64_t b0 = 0; b0 < B; b0 += e->max_batch) {
        const uint32_t nb = (uint32_t)std::min<uint64_t>(e->max_batch, B - b0);
        std::vector<uint32_t> lens(nb, (uint32_t)T);
        int rc = load_slots(e, ids + b0 * T, lens.data(), nb);
        if (rc) return rc;
        rc = prefill_impl(e, ids + b0 * T, lens.data(), nb, nullptr, nullptr, nullptr, targets + b0 * T, row_loss.data() + b0 * T);
        if (rc) return rc;
    }
    double total = 0.0;                                   // rows added in order, in double, as the reference does
    for (uint64_t i = 0; i < B * T; ++i)
        if (targets[i] >= 0) total += row_loss[i];
    *loss = (float)(total / (double)(num_valid ? num_valid : B * T));
    return SLLM_OK;
}

int sllm_sample(sllm_engine* e, const sllm_sampling* opt, const double* draws) {
    if (!e) return SLLM_ERR_INVALID;
    int rc = sampling_check(e, opt);
    if (rc) return rc;
    if (e->n_live == 0) return fail(e, SLLM_ERR_STATE, "sllm_sample: no live slots");
    if (opt->temperature > 0.0f && !draws) return fail(e, SLLM_ERR_INVALID, "sllm_sample: draws required when temperature > 0");
    const double* dd = nullptr;
    if (draws && opt->temperature > 0.0f) {
        rc = upload_draws(e, draws, e->n_live, 1, false);
        if (rc) return rc;
        dd = e->d_draws;
        CU(cudaMemsetAsync(e->st.draw_idx, 0, e->n_live * sizeof(int), e->stream));
    }
    rc = grow_for_step(e);
    if (rc) return rc;
    SampleArgs s = make_sample_args(e, opt, e->n_live, dd, 1, 0);
    rc = launch_sampler(e, s, false);
    if (rc) return rc;
    bool all_done, nonfinite;
    rc = check_finished_flags(e, &all_done, &nonfinite);
    if (rc) return rc;
    if (nonfinite) return fail(e, SLLM_ERR_NONFINITE, "Inference::generate: all logits are non-finite");
    return SLLM_OK;
}

int sllm_decode_step(sllm_engine* e) {
    if (!e) return SLLM_ERR_INVALID;
    if (e->n_live == 0) return fail(e, SLLM_ERR_STATE, "sllm_decode_step: no live slots");
    int rc = refresh_attn_order(e);
    if (rc) return rc;
    CU(cudaEventRecord(e->ev0, e->stream));
    rc = run_pass(e, decode_view(e), nullptr, e->n_live, e->step_logits, false);
    if (rc) return rc;
    CU(cudaEventRecord(e->ev1, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    cudaEventElapsedTime(&e->last_step_ms, e->ev0, e->ev1);
    e->decode_steps += 1;
    return check_status(e);
}

int sllm_get_step_logits(sllm_engine* e, uint32_t slot, float* host) {
    if (!e || !host || slot >= (uint32_t)e->max_batch) return fail(e, SLLM_ERR_INVALID, "sllm_get_step_logits: bad argument");
    CU(cudaMemcpyAsync(host, e->step_logits + (size_t)slot * e->md.V, (size_t)e->md.V * 4, cudaMemcpyDeviceToHost, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    return SLLM_OK;
}

int sllm_set_step_logits(sllm_engine* e, uint32_t slot, const float* host) {
    if (!e || !host || slot >= (uint32_t)e->max_batch) return fail(e, SLLM_ERR_INVALID, "sllm_set_step_logits: bad argument");
    CU(cudaMemcpyAsync(e->step_logits + (size_t)slot * e->md.V, host, (size_t)e->md.V * 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    return SLLM_OK;
}

int sllm_get_tokens(sllm_engine* e, uint32_t slot, uint32_t* out, uint64_t capacity, uint64_t* n) {
    if (!e || !n || slot >= (uint32_t)e->max_batch) return fail(e, SLLM_ERR_INVALID, "sllm_get_tokens: bad argument");
    int nt = 0;
    CU(cudaMemcpyAsync(&nt, e->st.n_tok + slot, 4, cudaMemcpyDeviceToHost, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    *n = (uint64_t)nt;
    if (out) {
        const size_t c = std::min<uint64_t>(capacity, (uint64_t)nt);
        CU(cudaMemcpyAsync(out, e->st.tokens + (size_t)slot * e->st.tok_cap, c * 4, cudaMemcpyDeviceToHost, e->stream));
        CU(cudaStreamSynchronize(e->stream));
    }
    return SLLM_OK;
}

int sllm_force_token(sllm_engine* e, uint32_t slot, uint32_t token) {
    if (!e || slot >= (uint32_t)e->n_live) return fail(e, SLLM_ERR_INVALID, "sllm_force_token: bad slot");
    if (token >= (uint32_t)e->md.V) return fail(e, SLLM_ERR_INVALID, "token id outside the vocabulary");
    int nt = 0;
    CU(cudaMemcpyAsync(&nt, e->st.n_tok + slot, 4, cudaMemcpyDeviceToHost, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    if (nt < 1) return fail(e, SLLM_ERR_STATE, "sllm_force_token: empty slot");
    const int words = e->md.V / 32;
    std::vector<uint32_t> toks(nt), seen(words, 0);
    CU(cudaMemcpyAsync(toks.data(), e->st.tokens + (size_t)slot * e->st.tok_cap, (size_t)nt * 4, cudaMemcpyDeviceToHost, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    toks[nt - 1] = token;
    for (uint32_t id : toks) seen[id >> 5] |= 1u << (id & 31);
    const int zero = 0;
    CU(cudaMemcpyAsync(e->st.seen + (size_t)slot * words, seen.data(), words * 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaMemcpyAsync(e->st.tokens + (size_t)slot * e->st.tok_cap + (nt - 1), &token, 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaMemcpyAsync(e->d_dec_id + slot, &token, 4, cudaMemcpyHostToDevice, e->stream));
    if (nt <= e->md.ctx) CU(cudaMemcpyAsync(e->st.finished + slot, &zero, 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    return SLLM_OK;
}

int sllm_truncate(sllm_engine* e, uint32_t slot, uint64_t n_tokens) {
    if (!e || slot >= (uint32_t)e->n_live) return fail(e, SLLM_ERR_INVALID, "sllm_truncate: bad slot");
    const int cap = e->st.tok_cap, V = e->md.V, words = V / 32;
    int nt = 0;
    CU(cudaMemcpyAsync(&nt, e->st.n_tok + slot, 4, cudaMemcpyDeviceToHost, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    if (n_tokens < 1 || n_tokens > (uint64_t)nt) return fail(e, SLLM_ERR_INVALID, "sllm_truncate: length out of range");
    std::vector<uint32_t> toks(n_tokens), seen(words, 0);
    CU(cudaMemcpyAsync(toks.data(), e->st.tokens + (size_t)slot * cap, n_tokens * 4, cudaMemcpyDeviceToHost, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    for (uint32_t id : toks) seen[id >> 5] |= 1u << (id & 31);
    const int n = (int)n_tokens, zero = 0, pos = n - 1;
    const int slot_i = (int)slot;
    CU(cudaMemcpyAsync(e->st.seen + (size_t)slot * words, seen.data(), words * 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaMemcpyAsync(e->st.n_tok + slot, &n, 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaMemcpyAsync(e->st.finished + slot, &zero, 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaMemcpyAsync(e->st.draw_idx + slot, &zero, 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaMemcpyAsync(e->d_dec_id + slot, &toks[n - 1], 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaMemcpyAsync(e->d_dec_pos + slot, &pos, 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaMemcpyAsync(e->d_dec_slot + slot, &slot_i, 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    e->h_len_bound[slot] = n;
    return SLLM_OK;
}

// ---- single slots: the building blocks of continuous batching ---------------------------------------------
static int park_slot(sllm_engine* e, int slot) {          // idle slot: finished, spare page everywhere, harmless pass inputs
    release_slot(e, slot);
    e->slot_released[slot] = 1;
    std::vector<int> row(e->pages_per_seq, e->spare_page);
    const int one = 1, zero = 0; const uint32_t zid = 0;
    CU(cudaMemcpyAsync(e->d_block_table + (size_t)slot * e->pages_per_seq, row.data(), row.size() * sizeof(int), cudaMemcpyHostToDevice, e->stream));
    CU(cudaMemcpyAsync(e->st.finished + slot, &one, 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaMemcpyAsync(e->st.n_tok + slot, &one, 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaMemcpyAsync(e->d_dec_slot + slot, &slot, 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaMemcpyAsync(e->d_dec_pos + slot, &zero, 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaMemcpyAsync(e->d_dec_id + slot, &zid, 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    return SLLM_OK;
}

int sllm_slot_assign(sllm_engine* e, uint32_t slot, const uint32_t* ids, uint32_t len) {
    if (!e || !ids) return fail(e, SLLM_ERR_INVALID, "sllm_slot_assign: null argument");
    const ModelDims& m = e->md;
    if (slot >= (uint32_t)e->max_batch) return fail(e, SLLM_ERR_CAPACITY, "sllm_slot_assign: slot exceeds max_batch");
    if (len == 0) return fail(e, SLLM_ERR_INVALID, "Inference::generate: prompt encoded to zero tokens");
    if (len > (uint32_t)m.ctx) return fail(e, SLLM_ERR_INVALID, "Model::forward: seq_len exceeds context_length");
    for (uint32_t i = 0; i < len; ++i)
        if (ids[i] >= (uint32_t)m.V) return fail(e, SLLM_ERR_INVALID, "token id outside the vocabulary");
    for (int s = e->n_live; s < (int)slot; ++s) { int rc = park_slot(e, s); if (rc) return rc; }   // slots skipped over stay idle
    e->n_live = std::max(e->n_live, (int)slot + 1);
    release_slot(e, (int)slot);
    e->slot_released[slot] = 0;
    const int cap = e->st.tok_cap, words = m.V / 32;
    std::vector<uint32_t> toks(cap, 0), seen(words, 0);
    for (uint32_t i = 0; i < len; ++i) { toks[i] = ids[i]; seen[ids[i] >> 5] |= 1u << (ids[i] & 31); }
    const int n = (int)len, zero = 0;
    bool changed = false;
    e->h_len_bound[slot] = n;
    int rc = ensure_pages(e, (int)slot, n, &changed);
    if (rc) return rc;
    rc = upload_block_table(e, (int)slot);
    if (rc) return rc;
    CU(cudaMemcpyAsync(e->st.tokens + (size_t)slot * cap, toks.data(), (size_t)cap * 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaMemcpyAsync(e->st.seen + (size_t)slot * words, seen.data(), (size_t)words * 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaMemcpyAsync(e->st.n_tok + slot, &n, 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaMemcpyAsync(e->st.finished + slot, &zero, 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaMemcpyAsync(e->st.draw_idx + slot, &zero, 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    const int sl = (int)slot;
    return prefill_impl(e, ids, &len, 1, nullptr, &sl);
}

// Tokens appended behind a live slot's history: only the new ids (and the slot's last token, whose KV entry may
// not exist yet when the loop ended on a sampling step) run through the model; earlier positions are served
// from the slot's KV pages.
int sllm_slot_append(sllm_engine* e, uint32_t slot, const uint32_t* ids, uint32_t len) {
    if (!e || !ids) return fail(e, SLLM_ERR_INVALID, "sllm_slot_append: null argument");
    const ModelDims& m = e->md;
    if (slot >= (uint32_t)e->n_live || e->slot_released[slot]) return fail(e, SLLM_ERR_STATE, "sllm_slot_append: slot holds no sequence");
    if (len == 0) return fail(e, SLLM_ERR_INVALID, "sllm_slot_append: no tokens");
    for (uint32_t i = 0; i < len; ++i)
        if (ids[i] >= (uint32_t)m.V) return fail(e, SLLM_ERR_INVALID, "token id outside the vocabulary");
    int nt = 0;
    CU(cudaMemcpyAsync(&nt, e->st.n_tok + slot, 4, cudaMemcpyDeviceToHost, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    if (nt < 1) return fail(e, SLLM_ERR_STATE, "sllm_slot_append: empty slot");
    if ((uint64_t)nt + len > (uint64_t)m.ctx) return fail(e, SLLM_ERR_CAPACITY, "sllm_slot_append: history plus new tokens exceed context_length");
    const int cap = e->st.tok_cap, words = m.V / 32;
    std::vector<uint32_t> run(len + 1), seen(words);
    CU(cudaMemcpyAsync(run.data(), e->st.tokens + (size_t)slot * cap + (nt - 1), 4, cudaMemcpyDeviceToHost, e->stream));
    CU(cudaMemcpyAsync(seen.data(), e->st.seen + (size_t)slot * words, (size_t)words * 4, cudaMemcpyDeviceToHost, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    for (uint32_t i = 0; i < len; ++i) { run[i + 1] = ids[i]; seen[ids[i] >> 5] |= 1u << (ids[i] & 31); }
    const int n = nt + (int)len, zero = 0;
    bool changed = false;
    e->h_len_bound[slot] = n;
    int rc = ensure_pages(e, (int)slot, n, &changed);
    if (rc) return rc;
    rc = upload_block_table(e, (int)slot);
    if (rc) return rc;
    CU(cudaMemcpyAsync(e->st.tokens + (size_t)slot * cap + nt, ids, (size_t)len * 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaMemcpyAsync(e->st.seen + (size_t)slot * words, seen.data(), (size_t)words * 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaMemcpyAsync(e->st.n_tok + slot, &n, 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaMemcpyAsync(e->st.finished + slot, &zero, 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaMemcpyAsync(e->st.draw_idx + slot, &zero, 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    const int sl = (int)slot, pos0 = nt - 1;
    const uint32_t run_len = len + 1;
    return prefill_impl(e, run.data(), &run_len, 1, nullptr, &sl, &pos0);
}

int sllm_slot_release(sllm_engine* e, uint32_t slot) {
    if (!e || slot >= (uint32_t)e->max_batch) return fail(e, SLLM_ERR_INVALID, "sllm_slot_release: bad slot");
    if ((int)slot >= e->n_live) return SLLM_OK;
    int rc = park_slot(e, (int)slot);
    // the live range ends at the highest slot that holds a sequence
    while (e->n_live > 0 && e->slot_released[e->n_live - 1]) e->n_live -= 1;
    return rc;
}

uint32_t sllm_num_live(const sllm_engine* e) { return e ? (uint32_t)e->n_live : 0; }

int sllm_engine_make_current(sllm_engine* e) {
    if (!e) return SLLM_ERR_INVALID;
    CU(cudaSetDevice(e->dev));
    return SLLM_OK;
}

int sllm_get_finished(sllm_engine* e, int32_t* flags, uint32_t n) {
    if (!e || !flags || n > (uint32_t)e->max_batch) return fail(e, SLLM_ERR_INVALID, "sllm_get_finished: bad argument");
    CU(cudaMemcpyAsync(flags, e->st.finished, (size_t)n * 4, cudaMemcpyDeviceToHost, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    return SLLM_OK;
}

// n_steps x (sampler, model pass) on the device; slots must have step logits (after prefill).
static int decode_loop_impl(sllm_engine* e, uint64_t n_steps, const sllm_sampling* opt, const double* d_draws, int stride,
                            int seeded, bool last_pass, bool* all_done_out) {
    SampleArgs s = make_sample_args(e, opt, e->n_live, d_draws, stride, seeded);
    cudaGraphExec_t ge = nullptr, ge_multi[2] = {nullptr, nullptr};
    constexpr uint64_t kMulti[2] = {32, 8}, check_every = 64;  // both divide check_every
    int launches_one = 0, launches_multi[2] = {0, 0};
    { int rc = refresh_attn_order(e); if (rc) return rc; }
    if (e->opt.use_graph) {
        // graphs of 32 and of 8 iterations: inside a graph consecutive kernels are joined by programmatic edges, and the
        // batch-1 kernel carries the next sampling step's first two kernels
        for (int attempt = 0; attempt < 2; ++attempt) {           // inserting a graph may empty the cache (cleared past 32 entries): fetch again
            int rc = get_iteration_graph(e, s, 1, &ge);
            if (rc) return rc;
            launches_one = launches_per_iteration(e);
            for (int k = 0; k < 2; ++k) {
                ge_multi[k] = nullptr;
                if (n_steps > kMulti[k]) {
                    rc = get_iteration_graph(e, s, (int)kMulti[k], &ge_multi[k]);
                    if (rc) return rc;
                    launches_multi[k] = launches_per_iteration(e);
                }
            }
        }
    }
    const uint64_t full_steps = last_pass ? n_steps : n_steps - 1;     // the last step of a generate call only samples
    uint64_t i = 0;
    while (i < n_steps) {
        uint64_t done = 1;
        int m = -1;
        for (int k = 0; k < 2 && m < 0; ++k)
            if (ge_multi[k] && i % kMulti[k] == 0 && i + kMulti[k] <= full_steps) m = k;
        if (m >= 0) {
            for (uint64_t k = 0; k < kMulti[m]; ++k) { int rc = grow_for_step(e); if (rc) return rc; }
            CU(cudaGraphLaunch(ge_multi[m], e->stream));
            e->launches += launches_multi[m];
            e->decode_steps += kMulti[m];
            done = kMulti[m];
        } else {
            int rc = grow_for_step(e);
            if (rc) return rc;
            const bool final_one = (i + 1 == n_steps) && !last_pass;
            if (final_one) {
                rc = launch_sampler(e, s, false);
                if (rc) return rc;
            } else if (ge) {
                CU(cudaGraphLaunch(ge, e->stream));
                e->launches += launches_one;
            } else {
                rc = enqueue_iteration(e, s);
                if (rc) return rc;
            }
            e->decode_steps += final_one ? 0 : 1;
        }
        i += done;
        if (i % check_every == 0 || i == n_steps) {
            bool all_done, nonfinite;
            int rc = check_finished_flags(e, &all_done, &nonfinite);
            if (rc) return rc;
            if (nonfinite) return fail(e, SLLM_ERR_NONFINITE, "Inference::generate: all logits are non-finite");
            if (all_done_out) *all_done_out = all_done;
            if (all_done) break;
        }
    }
    return SLLM_OK;
}

int sllm_decode_loop(sllm_engine* e, uint64_t n_steps, const sllm_sampling* opt, const double* draws) {
    if (!e) return SLLM_ERR_INVALID;
    int rc = sampling_check(e, opt);
    if (rc) return rc;
    if (e->n_live == 0) return fail(e, SLLM_ERR_STATE, "sllm_decode_loop: no live slots");
    if (n_steps == 0) return SLLM_OK;
    const double* dd = nullptr;
    if (opt->temperature > 0.0f) {
        if (!draws) return fail(e, SLLM_ERR_INVALID, "sllm_decode_loop: draws required when temperature > 0");
        rc = upload_draws(e, draws, e->n_live, n_steps, true);
        if (rc) return rc;
        dd = e->d_draws;
        CU(cudaMemsetAsync(e->st.draw_idx, 0, e->n_live * sizeof(int), e->stream));
    }
    return decode_loop_impl(e, n_steps, opt, dd, (int)n_steps, 0, true, nullptr);
}

static int generate_impl(sllm_engine* e, const uint32_t* ids, const uint32_t* lens, uint32_t n_seq, uint64_t max_new,
                         const sllm_sampling* opt, const double* draws, uint32_t* out, uint64_t out_stride, uint64_t* out_lens) {
    if (!e || !ids || !lens || !out || !out_lens) return fail(e, SLLM_ERR_INVALID, "sllm_generate: null argument");
    int rc = sampling_check(e, opt);
    if (rc) return rc;
    // A slot's token buffer holds 2 * context_length + 2 ids: a request that could outgrow it is refused here rather
    // than cut short without notice (the reference slides its window without bound).
    for (uint32_t s = 0; s < n_seq && s < (uint32_t)e->max_batch; ++s)
        if (lens[s] < (uint32_t)e->st.tok_cap && (uint64_t)lens[s] + max_new > (uint64_t)e->st.tok_cap)    // longer prompts: refused below
            return fail(e, SLLM_ERR_CAPACITY, "sllm_generate: prompt plus max_new_tokens exceed a slot's token buffer "
                                              "(2 * context_length + 2)");
    rc = load_slots(e, ids, lens, n_seq, /*allow_long=*/true);
    if (rc) return rc;
    if (max_new > 0) {
        const ModelDims& m = e->md;
        const double* dd = nullptr;
        int seeded = 0;
        if (opt->temperature > 0.0f) {
            if (draws) {
                rc = upload_draws(e, draws, n_seq, max_new, true);
            } else {
                seeded = 1;
                std::vector<double> t((size_t)n_seq * max_new);
                for (uint32_t s = 0; s < n_seq; ++s) canonical_stream(opt->seed + s, max_new, t.data() + (size_t)s * max_new);
                rc = upload_draws(e, t.data(), n_seq, max_new, false);
            }
            if (rc) return rc;
            dd = e->d_draws;
        }
        // prompts that fit the window are prefilled; longer ones start in the sliding phase below
        std::vector<uint32_t> fit_ids, fit_lens; std::vector<int> fit_slots;
        size_t off = 0;
        for (uint32_t s = 0; s < n_seq; ++s) {
            if (lens[s] <= (uint32_t)m.ctx) {
                fit_ids.insert(fit_ids.end(), ids + off, ids + off + lens[s]);
                fit_lens.push_back(lens[s]); fit_slots.push_back((int)s);
            }
            off += lens[s];
        }
        if (!fit_lens.empty()) {
            rc = prefill_impl(e, fit_ids.data(), fit_lens.data(), (uint32_t)fit_lens.size(), nullptr, fit_slots.data());
            if (rc) return rc;
            rc = decode_loop_impl(e, max_new, opt, dd, (int)max_new, seeded, false, nullptr);
            if (rc) return rc;
        }
        // The window slides (src/inference.cpp:40-48): once a slot holds more than context_length tokens,
        // every further token re-runs the last context_length tokens with positions restarting at 0, as
        // the reference does for every token.  Penalty history and draw cursor live on the device and carry on.
        SampleArgs sa = make_sample_args(e, opt, e->n_live, dd, (int)max_new, seeded);
        std::vector<int> h_ntok(n_seq), h_fin(n_seq);
        std::vector<uint32_t> window(m.ctx);
        for (;;) {
            CU(cudaMemcpyAsync(h_ntok.data(), e->st.n_tok, n_seq * 4, cudaMemcpyDeviceToHost, e->stream));
            CU(cudaMemcpyAsync(h_fin.data(), e->st.finished, n_seq * 4, cudaMemcpyDeviceToHost, e->stream));
            CU(cudaStreamSynchronize(e->stream));
            bool any = false;
            for (uint32_t s = 0; s < n_seq; ++s) {
                const uint64_t made = (uint64_t)h_ntok[s] - lens[s];
                if (h_fin[s] != 2 || made >= max_new || h_ntok[s] + 1 > e->st.tok_cap) continue;
                CU(cudaMemcpyAsync(window.data(), e->st.tokens + (size_t)s * e->st.tok_cap + (h_ntok[s] - m.ctx), (size_t)m.ctx * 4,
                                   cudaMemcpyDeviceToHost, e->stream));
                CU(cudaStreamSynchronize(e->stream));
                const uint32_t wl = (uint32_t)m.ctx; const int slot = (int)s, zero = 0;
                rc = prefill_impl(e, window.data(), &wl, 1, nullptr, &slot);
                if (rc) return rc;
                CU(cudaMemcpyAsync(e->st.finished + s, &zero, 4, cudaMemcpyHostToDevice, e->stream));
                any = true;
            }
            if (!any) break;
            rc = launch_sampler(e, sa, false);
            if (rc) return rc;
            bool all_done, nonfinite;
            rc = check_finished_flags(e, &all_done, &nonfinite);
            if (rc) return rc;
            if (nonfinite) return fail(e, SLLM_ERR_NONFINITE, "Inference::generate: all logits are non-finite");
        }
    }
    for (uint32_t s = 0; s < n_seq; ++s) {
        rc = sllm_get_tokens(e, s, out + (size_t)s * out_stride, out_stride, &out_lens[s]);
        if (rc) return rc;
    }
    return SLLM_OK;
}

// sllm_decode_loop with one CUDA event between consecutive iterations (each iteration is one graph replay):
// step_ms[i] = device time of iteration i.  For latency percentiles; the untimed loop replays 8 iterations per graph.
int sllm_decode_loop_timed(sllm_engine* e, uint64_t n_steps, const sllm_sampling* opt, const double* draws, float* step_ms) {
    if (!e || !step_ms) return fail(e, SLLM_ERR_INVALID, "sllm_decode_loop_timed: null argument");
    int rc = sampling_check(e, opt);
    if (rc) return rc;
    if (e->n_live == 0) return fail(e, SLLM_ERR_STATE, "sllm_decode_loop_timed: no live slots");
    if (n_steps == 0) return SLLM_OK;
    if (n_steps > 65536) return fail(e, SLLM_ERR_CAPACITY, "sllm_decode_loop_timed: at most 65536 steps per call");
    const double* dd = nullptr;
    if (opt->temperature > 0.0f) {
        if (!draws) return fail(e, SLLM_ERR_INVALID, "sllm_decode_loop_timed: draws required when temperature > 0");
        rc = upload_draws(e, draws, e->n_live, n_steps, true);
        if (rc) return rc;
        dd = e->d_draws;
        CU(cudaMemsetAsync(e->st.draw_idx, 0, e->n_live * sizeof(int), e->stream));
    }
    const SampleArgs s = make_sample_args(e, opt, e->n_live, dd, (int)n_steps, 0);
    rc = refresh_attn_order(e);
    if (rc) return rc;
    cudaGraphExec_t ge = nullptr;
    int per_iter = 0;
    if (e->opt.use_graph) {
        rc = get_iteration_graph(e, s, 1, &ge);
        if (rc) return rc;
        per_iter = launches_per_iteration(e);
    }
    while (e->step_events.size() < n_steps + 1) {
        cudaEvent_t ev = nullptr;
        CU(cudaEventCreate(&ev));
        e->step_events.push_back(ev);
    }
    for (uint64_t i = 0; i < n_steps; ++i) {
        rc = grow_for_step(e);
        if (rc) return rc;
        CU(cudaEventRecord(e->step_events[i], e->stream));
        if (ge) { CU(cudaGraphLaunch(ge, e->stream)); e->launches += per_iter; }
        else { rc = enqueue_iteration(e, s); if (rc) return rc; }
        e->decode_steps += 1;
    }
    CU(cudaEventRecord(e->step_events[n_steps], e->stream));
    bool all_done, nonfinite;
    rc = check_finished_flags(e, &all_done, &nonfinite);
    if (rc) return rc;
    if (nonfinite) return fail(e, SLLM_ERR_NONFINITE, "Inference::generate: all logits are non-finite");
    for (uint64_t i = 0; i < n_steps; ++i) CU(cudaEventElapsedTime(&step_ms[i], e->step_events[i], e->step_events[i + 1]));
    return SLLM_OK;
}

int sllm_generate(sllm_engine* e, const uint32_t* ids, const uint32_t* lens, uint32_t n_seq, uint64_t max_new,
                  const sllm_sampling* opt, const double* draws, uint32_t* out, uint64_t out_stride, uint64_t* out_lens) {
    try {
        return generate_impl(e, ids, lens, n_seq, max_new, opt, draws, out, out_stride, out_lens);
    } catch (const std::exception& ex) {            // host allocation failure: nothing may unwind through the C ABI
        return fail(e, SLLM_ERR_CAPACITY, std::string("sllm_generate: ") + ex.what());
    }
}

// ---- single-kernel entry points ------------------------------------------------------------------------------
namespace {

// Scratch of sllm_k_attn_decode_static: tickets | (max, sum) pairs | partial outputs.
constexpr int kStaticPairs = 64;                     // n_tok * heads
constexpr int kStaticHd = 128;
constexpr size_t kStaticTicketBytes = 256;           // 64 x u32
constexpr size_t kStaticMlBytes = (size_t)kStaticPairs * kMaxSplits * 2 * sizeof(float);
constexpr size_t kStaticOBytes = (size_t)kStaticPairs * kMaxSplits * kStaticHd * sizeof(float);
static __device__ __align__(256) unsigned char g_attn_static_scratch[kStaticTicketBytes + kStaticMlBytes + kStaticOBytes];

// device address of the array per device ordinal, looked up once with that device current
unsigned char* g_static_scratch_addr[64] = {};
std::mutex g_static_scratch_mutex;

int attn_decode_launch(sllm_engine* e, uint32_t layer, uint32_t n_tok, const float* d_q, const int32_t* d_slot,
                       const int32_t* d_pos, uint32_t n_splits, float* d_out, cudaStream_t stream, float* part_o,
                       float* part_ml, unsigned int* ticket) {
    const ModelDims& m = e->md;
    AttnDecArgs t{};
    t.q = d_q; t.out = d_out; t.out_bf16 = nullptr; t.m = m;
    t.kv = KvView{e->kv_pool, e->d_block_table, e->n_pages, e->pages_per_seq};
    t.pass = PassView{nullptr, d_slot, d_pos, (int)n_tok, nullptr, 0};
    t.layer = (int)layer;
    const int pages_per_split = (e->pages_per_seq + (int)n_splits - 1) / (int)n_splits;
    t.keys_per_split = pages_per_split * kPage;
    t.n_splits = (e->pages_per_seq + pages_per_split - 1) / pages_per_split;
    t.part_o = part_o; t.part_ml = part_ml; t.ticket = ticket;
    if ((int)n_tok > e->split_tok_cap) {
        // many tokens (n_splits is 1 here): the page-streaming kernel the engine itself uses at large batch
        cudaStream_t own = e->stream;
        e->stream = stream;
        const int rc = e->f32 ? launch_attn<float>(e, t, false) : launch_attn<__nv_bfloat16>(e, t, false);
        e->stream = own;
        return rc;
    }
    const dim3 grid(t.n_splits, m.H, n_tok), block(kAttnThreads);
    void (*kern)(AttnDecArgs) = nullptr;
    if (e->f32) {
        switch (m.hd) { case 16: kern = k_attn_decode<float, 16>; break; case 32: kern = k_attn_decode<float, 32>; break;
                        case 64: kern = k_attn_decode<float, 64>; break; case 128: kern = k_attn_decode<float, 128>; break; }
    } else {
        switch (m.hd) { case 16: kern = k_attn_decode<__nv_bfloat16, 16>; break; case 32: kern = k_attn_decode<__nv_bfloat16, 32>; break;
                        case 64: kern = k_attn_decode<__nv_bfloat16, 64>; break; case 128: kern = k_attn_decode<__nv_bfloat16, 128>; break; }
    }
    if (!kern) return fail(e, SLLM_ERR_INVALID, "unsupported head_dim");
    kern<<<grid, block, 0, stream>>>(t);
    CU(cudaGetLastError());
    e->launches += 1;
    return SLLM_OK;
}

int attn_args_check(sllm_engine* e, uint32_t layer, uint32_t n_tok, const void* q, const void* s, const void* p,
                    uint32_t n_splits, const void* out) {
    if (!e) return SLLM_ERR_INVALID;
    if (!q || !s || !p || !out) return fail(e, SLLM_ERR_INVALID, "attention kernel: null device pointer");
    if (layer >= (uint32_t)e->md.L) return fail(e, SLLM_ERR_INVALID, "attention kernel: layer out of range");
    if (n_tok == 0) return fail(e, SLLM_ERR_INVALID, "attention kernel: no tokens");
    if (n_splits < 1 || n_splits > (uint32_t)kMaxSplits) return fail(e, SLLM_ERR_INVALID, "attention kernel: n_splits must be 1..32");
    return SLLM_OK;
}

}  // namespace

int sllm_k_attn_decode(sllm_engine* e, uint32_t layer, uint32_t n_tok, const float* d_q, const int32_t* d_tok_slot,
                       const int32_t* d_tok_pos, uint32_t n_splits, float* d_out, void* stream) {
    int rc = attn_args_check(e, layer, n_tok, d_q, d_tok_slot, d_tok_pos, n_splits, d_out);
    if (rc) return rc;
    if (n_splits > 1 && n_tok > (uint32_t)e->split_tok_cap)
        return fail(e, SLLM_ERR_CAPACITY, "attention kernel: more than 64 tokens need n_splits = 1");
    return attn_decode_launch(e, layer, n_tok, d_q, d_tok_slot, d_tok_pos, n_splits, d_out,
                              stream ? (cudaStream_t)stream : e->stream, e->part_o, e->part_ml, e->ticket);
}

// Allocation-free variant: split-K scratch in the library's own device array (see sllm.h).
int sllm_k_attn_decode_static(sllm_engine* e, uint32_t layer, uint32_t n_tok, const float* d_q,
                              const int32_t* d_tok_slot, const int32_t* d_tok_pos, uint32_t n_splits, float* d_out,
                              void* stream) {
    int rc = attn_args_check(e, layer, n_tok, d_q, d_tok_slot, d_tok_pos, n_splits, d_out);
    if (rc) return rc;
    if ((uint64_t)n_tok * (uint64_t)e->md.H > (uint64_t)kStaticPairs || e->md.hd > kStaticHd)
        return fail(e, SLLM_ERR_CAPACITY, "sllm_k_attn_decode_static: request exceeds the fixed scratch (n_tok * num_heads <= 64, "
                                           "head_dim <= 128); use sllm_k_attn_decode");
    int cur = -1;
    CU(cudaGetDevice(&cur));
    if (cur != e->dev || cur < 0 || cur >= 64)
        return fail(e, SLLM_ERR_STATE, "sllm_k_attn_decode_static: the engine's device must be the current device");
    std::lock_guard<std::mutex> guard(g_static_scratch_mutex);      // the table is shared by every engine of the process
    if (!g_static_scratch_addr[cur]) {
        // The array's name is only a host-side handle: the kernel needs the address the symbol has on
        // THIS device, which the runtime reports once the device is current.
        void* p = nullptr;
        CU(cudaGetSymbolAddress(&p, g_attn_static_scratch));
        if (!p) return fail(e, SLLM_ERR_CUDA, "sllm_k_attn_decode_static: no device address for the scratch array");
        g_static_scratch_addr[cur] = static_cast<unsigned char*>(p);
    }
    unsigned char* base = g_static_scratch_addr[cur];
    cudaStream_t st = stream ? (cudaStream_t)stream : e->stream;
    // tickets must start at zero; partial results are fully rewritten before they are read
    CU(cudaMemsetAsync(base, 0, kStaticTicketBytes, st));
    return attn_decode_launch(e, layer, n_tok, d_q, d_tok_slot, d_tok_pos, n_splits, d_out, st,
                              reinterpret_cast<float*>(base + kStaticTicketBytes + kStaticMlBytes),
                              reinterpret_cast<float*>(base + kStaticTicketBytes),
                              reinterpret_cast<unsigned int*>(base));
}

extern "C++" {
namespace {
// K/V rows of one slot between the host ([n_pos][num_heads * head_dim] fp32) and the paged cache (cache element type).
template <typename KVT, bool WRITE>
__global__ void __launch_bounds__(256) k_kv_rows(KvView kv, ModelDims m, int layer, int slot, int pos0, float* k_rows, float* v_rows) {
    const int p = pos0 + blockIdx.x;
    const int page = kv.block_table[(size_t)slot * kv.pages_per_seq + p / kPage];
    for (int c = threadIdx.x; c < m.D; c += blockDim.x) {
        const int h = c / m.hd, d = c % m.hd;
        KVT* kp = kv_ptr<KVT>(kv, m, layer, page, 0, h, p % kPage) + d;
        KVT* vp = kv_ptr<KVT>(kv, m, layer, page, 1, h, p % kPage) + d;
        const size_t i = (size_t)blockIdx.x * m.D + c;
        if (WRITE) { *kp = from_float<KVT>(k_rows[i]); *vp = from_float<KVT>(v_rows[i]); }
        else { k_rows[i] = to_float(*kp); v_rows[i] = to_float(*vp); }
    }
}

int kv_rows_impl(sllm_engine* e, uint32_t layer, uint32_t slot, uint32_t pos0, uint32_t n_pos, float* k, float* v, bool write) {
    if (!e || !k || !v) return fail(e, SLLM_ERR_INVALID, "sllm_kv_rows: null argument");
    const ModelDims& m = e->md;
    if (layer >= (uint32_t)m.L) return fail(e, SLLM_ERR_INVALID, "sllm_kv_rows: layer out of range");
    if (slot >= (uint32_t)e->n_live || e->slot_released[slot]) return fail(e, SLLM_ERR_STATE, "sllm_kv_rows: slot holds no sequence");
    if (n_pos == 0) return SLLM_OK;
    if ((uint64_t)pos0 + n_pos > (uint64_t)e->slot_pages[slot].size() * kPage)
        return fail(e, SLLM_ERR_INVALID, "sllm_kv_rows: positions beyond the pages the slot holds");
    const KvView kv{e->kv_pool, e->d_block_table, e->n_pages, e->pages_per_seq};
    // staged through the pass buffers q (K rows) and att (V rows), a pass's worth of positions at a time
    for (uint32_t b = 0; b < n_pos; b += (uint32_t)e->pass_cap) {
        const uint32_t n = std::min<uint32_t>((uint32_t)e->pass_cap, n_pos - b);
        const size_t bytes = (size_t)n * m.D * sizeof(float), off = (size_t)b * m.D;
        if (write) {
            CU(cudaMemcpyAsync(e->q, k + off, bytes, cudaMemcpyHostToDevice, e->stream));
            CU(cudaMemcpyAsync(e->att, v + off, bytes, cudaMemcpyHostToDevice, e->stream));
        }
        const int p0 = (int)(pos0 + b);
        if (e->f32) {
            if (write) k_kv_rows<float, true><<<n, 256, 0, e->stream>>>(kv, m, (int)layer, (int)slot, p0, e->q, e->att);
            else k_kv_rows<float, false><<<n, 256, 0, e->stream>>>(kv, m, (int)layer, (int)slot, p0, e->q, e->att);
        } else {
            if (write) k_kv_rows<__nv_bfloat16, true><<<n, 256, 0, e->stream>>>(kv, m, (int)layer, (int)slot, p0, e->q, e->att);
            else k_kv_rows<__nv_bfloat16, false><<<n, 256, 0, e->stream>>>(kv, m, (int)layer, (int)slot, p0, e->q, e->att);
        }
        CU(cudaGetLastError());
        e->launches += 1;
        if (!write) {
            CU(cudaMemcpyAsync(k + off, e->q, bytes, cudaMemcpyDeviceToHost, e->stream));
            CU(cudaMemcpyAsync(v + off, e->att, bytes, cudaMemcpyDeviceToHost, e->stream));
        }
        CU(cudaStreamSynchronize(e->stream));
    }
    return SLLM_OK;
}

// A block whose only thread waits on an mbarrier that nothing ever arrives at: the wait runs out after limit_ns, the
// block raises the status word and returns.
__global__ void k_wait_probe(unsigned long long limit_ns, unsigned int* status) {
    __shared__ __align__(8) unsigned long long bar;
    const uint32_t b = (uint32_t)__cvta_generic_to_shared(&bar);
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(b));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (!mbar_wait_bounded(b, 0, limit_ns)) atomicExch(status, 90u);
}
}  // namespace
}  // extern "C++"

int sllm_kv_write(sllm_engine* e, uint32_t layer, uint32_t slot, uint32_t pos0, uint32_t n_pos, const float* k_rows, const float* v_rows) {
    return kv_rows_impl(e, layer, slot, pos0, n_pos, const_cast<float*>(k_rows), const_cast<float*>(v_rows), true);
}
int sllm_kv_read(sllm_engine* e, uint32_t layer, uint32_t slot, uint32_t pos0, uint32_t n_pos, float* k_rows, float* v_rows) {
    return kv_rows_impl(e, layer, slot, pos0, n_pos, k_rows, v_rows, false);
}

int sllm_k_wait_probe(sllm_engine* e, uint32_t limit_us) {
    if (!e) return SLLM_ERR_INVALID;
    if (limit_us == 0 || limit_us > 100000) return fail(e, SLLM_ERR_INVALID, "sllm_k_wait_probe: limit must be 1..100000 microseconds");
    k_wait_probe<<<1, 1, 0, e->stream>>>((unsigned long long)limit_us * 1000ull, e->d_status);
    CU(cudaGetLastError());
    e->launches += 1;
    return check_status(e);
}

#ifdef SLLM_TIMELINE
// debug builds only: copy out and reset the device-side timeline (pairs of id, globaltimer ns)
int sllm_debug_timeline(unsigned long long* host, unsigned int cap_pairs, unsigned int* n) {
    unsigned int cnt = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&cnt, g_tl_n, 4) != cudaSuccess) return SLLM_ERR_CUDA;
    if (cnt > (1u << 15)) cnt = 1u << 15;
    if (cnt > cap_pairs) cnt = cap_pairs;
    if (cnt && cudaMemcpyFromSymbol(host, g_tl_buf, (size_t)cnt * 16) != cudaSuccess) return SLLM_ERR_CUDA;
    cudaMemcpyToSymbol(g_tl_n, &zero, 4);
    *n = cnt;
    return SLLM_OK;
}
#endif

}  // extern "C"

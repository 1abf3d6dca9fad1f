// dn_seq.cu -- C ABI of libdnet_b200_seq.so (include/dnet_b200_seq.h): host bookkeeping of the batched step --
// bound weight pointers, the page pool and the state slots, the staging of a step's batch description, and the
// launch sequence of a layer.  All arithmetic is in dn_seq_kernels.cuh.
#include "dn_seq_kernels.cuh"
#include "dn_seq_recur.cuh"
#include "dn_seq_moe.cuh"
#include "dn_seq_latent.cuh"
#include "dn_seq_gdelta.cuh"
#include "dn_gemm_tc.cuh"      // the tcgen05 / TMA GEMM the llama-family prefill runs on (namespace dn)
#include "../../include/dnet_b200_seq.h"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <new>
#include <type_traits>
#include <vector>

using namespace dnseq;

#define DN_OK 0
#define DN_EINVAL (-22)
#define DN_ENOMEM (-12)
#define DN_ENOENT (-2)
#define DN_ECUDA (-5)
#define DN_ENOSPC (-28)

static thread_local char g_err[512] = "";
static int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
#define CK(...)                                                                                                 \
  do {                                                                                                          \
    cudaError_t e_ = (__VA_ARGS__);                                                                             \
    if (e_ != cudaSuccess)                                                                                      \
      return fail(DN_ECUDA, "%s failed: %s (%s:%d)", #__VA_ARGS__, cudaGetErrorString(e_), __FILE__, __LINE__); \
  } while (0)

static std::atomic<long long> g_launches{0};
static int g_device = -1;
static int g_sms = 0;
static size_t g_max_smem = 0;

// weight matrices and the activation buffers they multiply get TMA descriptors in bf16 mode
struct XMaps {
  CUtensorMap m[3];     // token tiles of 32 / 64 / 128 rows
  bool ok = false;
};
struct SeqLayer {
  dn_seq_layer_cfg c;
  const void* w[DN_SQ_COUNT];
  CUtensorMap tm[DN_SQ_COUNT];
  bool tm_ok[DN_SQ_COUNT];
  XMaps x_mo, x_act;            // the mixer's output buffer [MB, Co] and the feed-forward's [MB, ff]
  XMaps x_mo_r, x_lr;           // the linear-attention half's [MB, Rv]; the decay projection's inner [MB, rank]
  int Cq, Ck, Cv, Co;           // projection widths: q, k, v and the mixer's output before W_o
  int Rc, Rv;                   // linear-attention half of a parallel mixer: q / k width, v / output width
  int Cql, Col;                 // latent attention: widths of the absorbed queries [H (R + rot)] and of the output in latent space [H R]
  float* inv_freq;              // [rot/2] device
  std::vector<const void*> etab_h;   // routed experts: [3][E] gate, up, down
  const void** etab_d;
  CUtensorMap* emaps_d;              // [3][E] TMA descriptors of the experts' matrices, in device memory (bf16 mode)
  std::vector<char> emap_ok;
  CUtensorMap x_eact[2];             // the experts' activations [pairs, ff], 64- and 128-row boxes
  bool x_eact_ok;
};
// One run of a layer.  A layer inside the loop runs loop_times times on the same weights; every run has its own
// pages, carried inputs and recurrent state.
struct Run {
  int layer;
  bool inject;                  // a pass of the loop starts here: x <- W_in [x; x0] first
  int kv_index;                 // attention: which page pool (own or the one it borrows); -1 without attention
  size_t conv_off, state_off;   // element offsets into a slot's carried inputs (conv taps, shifted row) / fp32 state
  size_t canon_off[2];          // ... and of the carried rows of the two sublayers' input convolutions
};

struct dn_seq_model {
  dn_seq_cfg cfg;
  std::vector<SeqLayer> L;
  std::vector<Run> runs;
  const void *embed = nullptr, *final_norm = nullptr, *head = nullptr;
  const void* mw[16] = {nullptr};     // the other model tensors, by (which - DN_SQ_EMBED)
  CUtensorMap tm_loop_in, x_xg[2];    // x_xg: the tokens' rows sorted by expert [pairs, W], 64- and 128-row boxes
  bool tm_loop_ok = false, x_xg_ok = false;
  void* xg = nullptr;
  float* attn_part = nullptr;         // partials of split attention rows [AT_SPLIT_ROWS][heads][AT_MAX_SPLITS][2 + vdim padded]
  XMaps x_cat, x_xm[SHIFT_MAX];
  size_t esz = 2;
  int S1 = 1, MB = 0, max_pages = 0;
  // scratch
  float *xs = nullptr, *y = nullptr, *pa = nullptr, *pb = nullptr, *qn = nullptr, *kn = nullptr, *vv = nullptr, *od = nullptr,
        *beta = nullptr, *decay = nullptr, *y2 = nullptr, *x0 = nullptr, *dz = nullptr, *rwt = nullptr, *eo = nullptr, *sgate = nullptr;
  int part_dv = 256;            // widest value row (padded to 32) of a split attention row's partials
  void *h = nullptr, *uq = nullptr, *uk = nullptr, *uv = nullptr, *qb = nullptr, *mo = nullptr, *gt = nullptr, *act = nullptr, *cat = nullptr,
       *xm = nullptr, *lr = nullptr, *eact = nullptr;
  int32_t *ridx = nullptr, *rpos = nullptr, *rtok = nullptr, *tiles = nullptr;
  int max_tiles = 0;
  // state
  std::vector<void*> kpool, vpool;
  std::vector<void*> pkpool, pvpool;     // mean-pooled blocks behind a sliding window: [pages][pool_rows][row] (null: the run has none)
  std::vector<int> last_tok;             // per slot: the sequence's last token (-1: none yet), for the bigram row
  void* hn = nullptr;                    // the normed rows before the sublayer's input convolution [MB, W]
  float *un = nullptr, *aun = nullptr;   // generalized delta rule: unit keys, removal rate times unit key [MB, C]
  void* conv_state = nullptr;
  size_t conv_stride = 0;       // elements per slot
  float* delta_state = nullptr;
  size_t delta_stride = 0;
  std::vector<int> free_pages, free_slots;
  std::vector<std::vector<int>> pages;   // per slot
  std::vector<int> length;               // per slot, -1: closed
  XMaps x_h;                    // the normed activations [MB, W]
  CUtensorMap tm_head;
  bool tm_head_ok = false;
  unsigned int* tc_err = nullptr;   // set by a bounded in-kernel wait of the tcgen05 GEMM that ran out
  // decode steps (every entry brings one token) replay a captured graph per (entries, wanted rows): all kernel
  // arguments of such a step are fixed buffers, the batch description is read from the staging area
  bool graphs_on = true;
  std::map<std::pair<int, int>, std::pair<cudaGraphExec_t, long long>> graphs;   // -> (exec, kernels per replay)
  float* lg_buf = nullptr;          // [8][vocab] logits of a replayed step, copied to the caller's buffer
  // phase profiler (off by default): one event at every phase boundary of a step, read back by dn_seq_profile_read
  bool prof_on = false;
  std::vector<cudaEvent_t> prof_pool;
  std::vector<std::pair<int, cudaEvent_t>> prof_marks;
  double prof_ms[DN_SEQ_PH_COUNT] = {0};
  // staging
  int32_t *stage_h = nullptr, *stage_d = nullptr, *bt_h = nullptr, *bt_d = nullptr;
  size_t stage_ints = 0;
  cudaEvent_t staged = nullptr;
};

template <typename... KArgs, typename... Args>
static cudaError_t launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
  g_launches++;
  kern<<<grid, block, smem, s>>>(static_cast<KArgs>(args)...);
  return cudaGetLastError();
}

extern "C" const char* dn_seq_last_error(void) { return g_err; }
extern "C" int64_t dn_seq_launch_count(void) { return (int64_t)g_launches.load(); }

extern "C" int dn_seq_init(int device) {
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0)
    return fail(DN_ECUDA, "no CUDA device visible (%s): libdnet_b200_seq has no CPU fallback", cudaGetErrorString(e));
  if (device < 0 || device >= n) return fail(DN_EINVAL, "device %d out of range [0,%d)", device, n);
  CK(cudaSetDevice(device));
  cudaDeviceProp p;
  CK(cudaGetDeviceProperties(&p, device));
  if (p.major != 10) return fail(DN_EINVAL, "device %d is sm_%d%d; this library is built for sm_100a only", device, p.major, p.minor);
  g_sms = p.multiProcessorCount;
  g_max_smem = p.sharedMemPerBlockOptin;
  g_device = device;
  return DN_OK;
}

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static PFN_encodeTiled g_encode = nullptr;
// [rows, cols] bf16 row-major, box box_rows x 64 columns (one 128-byte swizzle span); false when the tensor cannot
// have one (pitch or base not a multiple of 16 bytes) -- such products run on the CUDA-core kernels
static bool make_tmap(CUtensorMap* out, const void* base, int rows, int cols, int box_rows) {
  if (!g_encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
      return false;
    g_encode = (PFN_encodeTiled)fn;
  }
  if (!base || cols % 64 || ((uintptr_t)base & 15)) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return g_encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
static void make_xmaps(XMaps* x, const void* base, int rows, int cols) {
  x->ok = true;
  const int br[3] = {32, 64, 128};
  for (int i = 0; i < 3; i++) x->ok = x->ok && make_tmap(&x->m[i], base, rows, cols, br[i]);
}

template <class P>
static int dalloc(P** p, size_t bytes) {
  void* q = nullptr;
  if (cudaMalloc(&q, bytes ? bytes : 16) != cudaSuccess) return fail(DN_ENOMEM, "cudaMalloc of %zu bytes failed", bytes);
  *p = (P*)q;
  return DN_OK;
}

extern "C" int dn_seq_model_destroy(dn_seq_model* m) {
  if (!m) return DN_OK;
  cudaDeviceSynchronize();
  void* ptrs[] = {m->xs, m->y, m->pa, m->pb, m->qn, m->kn, m->vv, m->od, m->beta, m->decay, m->h, m->uq, m->uk, m->uv, m->qb,
                  m->mo, m->gt, m->act, m->conv_state, m->delta_state, m->stage_d, m->bt_d, m->tc_err, m->y2, m->x0, m->dz, m->rwt,
                  m->eo, m->cat, m->xm, m->lr, m->eact, m->ridx, m->rpos, m->rtok, m->tiles, m->xg, m->attn_part, m->sgate, m->hn, m->un, m->aun};
  for (void* p : ptrs) if (p) cudaFree(p);
  for (auto& g : m->graphs) cudaGraphExecDestroy(g.second.first);
  if (m->lg_buf) cudaFree(m->lg_buf);
  for (auto& pm : m->prof_marks) cudaEventDestroy(pm.second);
  for (cudaEvent_t ev : m->prof_pool) cudaEventDestroy(ev);
  for (void* p : m->kpool) if (p) cudaFree(p);
  for (void* p : m->vpool) if (p) cudaFree(p);
  for (void* p : m->pkpool) if (p) cudaFree(p);
  for (void* p : m->pvpool) if (p) cudaFree(p);
  for (auto& l : m->L) { if (l.inv_freq) cudaFree(l.inv_freq); if (l.etab_d) cudaFree((void*)l.etab_d); if (l.emaps_d) cudaFree(l.emaps_d); }
  if (m->stage_h) cudaFreeHost(m->stage_h);
  if (m->bt_h) cudaFreeHost(m->bt_h);
  if (m->staged) cudaEventDestroy(m->staged);
  delete m;
  return DN_OK;
}

extern "C" int dn_seq_model_create(const dn_seq_cfg* cfg, const dn_seq_layer_cfg* layers, dn_seq_model** out) {
  if (!cfg || !layers || !out) return fail(DN_EINVAL, "null argument");
  if (g_device < 0) return fail(DN_EINVAL, "dn_seq_init() has not been called");
  if (cfg->width <= 0 || cfg->vocab <= 0 || cfg->n_layers <= 0) return fail(DN_EINVAL, "width / vocab / n_layers must be positive");
  if (cfg->streams < 0 || cfg->streams > MAX_STREAMS) return fail(DN_EINVAL, "streams %d unsupported (0..%d)", cfg->streams, MAX_STREAMS);
  if (cfg->dtype != DN_SEQ_BF16 && cfg->dtype != DN_SEQ_F32) return fail(DN_EINVAL, "dtype %d unsupported", cfg->dtype);
  if (cfg->pool_pages <= 0 || cfg->max_seqs <= 0 || cfg->max_batch_tokens <= 0) return fail(DN_EINVAL, "pool / slots / batch must be positive");
  dn_seq_model* m = new (std::nothrow) dn_seq_model();
  if (!m) return fail(DN_ENOMEM, "out of host memory");
  m->cfg = *cfg;
  m->esz = cfg->dtype == DN_SEQ_F32 ? 4 : 2;
  m->S1 = cfg->streams > 0 ? cfg->streams : 1;
  m->MB = cfg->max_batch_tokens;
  m->max_pages = cfg->pool_pages;
  m->L.resize(cfg->n_layers);
  int mq = 1, mk = 1, mv = 1, mo = 1, mh = 1, mff = 1, mdq = 1, mrank = 1, mpairs = 0, meff = 1, mexp = 1;
  bool any_wkv = false, any_gdelta = false;
  int rc = DN_OK;
  const bool looped = cfg->loop_times > 0;
  if (looped && (cfg->loop_start < 0 || cfg->loop_stop > cfg->n_layers || cfg->loop_start >= cfg->loop_stop))
    rc = fail(DN_EINVAL, "loop [%d, %d) x %d does not fit %d layers", cfg->loop_start, cfg->loop_stop, cfg->loop_times, cfg->n_layers);
  if (rc == DN_OK && cfg->norm_kind != DN_NORM_RMS && cfg->norm_kind != DN_NORM_DYT && cfg->norm_kind != DN_NORM_LAYER) rc = fail(DN_EINVAL, "norm kind %d unknown", cfg->norm_kind);
  if (rc == DN_OK && cfg->norm_kind != DN_NORM_DYT && cfg->embed_norm) rc = fail(DN_EINVAL, "a norm on the embedding exists as dynamic tanh only");
  if (rc == DN_OK && cfg->norm_kind == DN_NORM_LAYER && (cfg->post_norm || cfg->no_pre_norm)) rc = fail(DN_EINVAL, "layer norms stand before the sublayers only");
  if (rc == DN_OK && (cfg->canon_taps < 0 || cfg->canon_taps > 9 || (cfg->canon_taps > 0 && (cfg->no_pre_norm || cfg->norm_kind == DN_NORM_DYT || cfg->loop_times > 0))))
    rc = fail(DN_EINVAL, "input convolutions of %d taps unsupported (0..9, behind an RMS or layer norm before the sublayer, no loop)", cfg->canon_taps);
  if (rc == DN_OK && (cfg->bigram_buckets < 0 || (cfg->bigram_buckets > 0 && (cfg->bigram_mul_prev < 0 || cfg->bigram_mul_cur < 0))))
    rc = fail(DN_EINVAL, "bigram table of %d buckets with multipliers %d / %d unsupported", cfg->bigram_buckets, cfg->bigram_mul_prev, cfg->bigram_mul_cur);
  if (rc == DN_OK && cfg->norm_kind == DN_NORM_RMS && cfg->post_norm && cfg->streams > 0)
    rc = fail(DN_EINVAL, "an RMS norm after a sublayer joins the plain residual only (streams = 0)");
  for (int i = 0; i < cfg->n_layers && rc == DN_OK; i++) {
    SeqLayer& l = m->L[i];
    l.c = layers[i];
    memset(l.w, 0, sizeof(l.w));
    memset(l.tm_ok, 0, sizeof(l.tm_ok));
    l.inv_freq = nullptr;
    l.etab_d = nullptr;
    l.emaps_d = nullptr;
    l.x_eact_ok = false;
    l.Rc = l.Rv = l.Cql = l.Col = 0;
    const dn_seq_layer_cfg& c = l.c;
    if (c.heads <= 0 || c.kv_heads <= 0 || c.heads % c.kv_heads || c.dim <= 0 || c.vdim <= 0) {
      rc = fail(DN_EINVAL, "layer %d: heads %d / kv_heads %d / dim %d / vdim %d unsupported", i, c.heads, c.kv_heads, c.dim, c.vdim);
      break;
    }
    if (c.conv < 0 || c.conv > 9) { rc = fail(DN_EINVAL, "layer %d: conv taps %d unsupported (0..9)", i, c.conv); break; }
    if (c.mixer == DN_MIX_ATTENTION || c.mixer == DN_MIX_PARALLEL) {
      if (c.vdim > 256) { rc = fail(DN_EINVAL, "layer %d: vdim %d > 256", i, c.vdim); break; }
      if (c.rot_dims < 0 || c.rot_dims > c.dim || (c.rot_dims & 1)) { rc = fail(DN_EINVAL, "layer %d: rot dims %d unsupported", i, c.rot_dims); break; }
      l.Cq = c.heads * c.dim;
      l.Co = c.heads * c.vdim;
      if (c.kv_from >= 0) {
        if (c.kv_from >= i || m->L[c.kv_from].c.mixer != DN_MIX_ATTENTION || m->L[c.kv_from].c.kv_from >= 0 ||
            m->L[c.kv_from].c.kv_heads != c.kv_heads || m->L[c.kv_from].c.dim != c.dim || m->L[c.kv_from].c.vdim != c.vdim) {
          rc = fail(DN_EINVAL, "layer %d: kv_from %d must name an earlier attention layer with its own keys and the same head sizes", i, c.kv_from);
          break;
        }
        l.Ck = l.Cv = 0;
      } else {
        l.Ck = c.kv_heads * c.dim;
        l.Cv = c.kv_heads * c.vdim;
      }
      if (c.v_is_k) {
        if (c.vdim != c.dim || c.kv_from >= 0 || c.conv > 0) { rc = fail(DN_EINVAL, "layer %d: values that are the keys need vdim = dim, own keys and no convolutions", i); break; }
        l.Cv = 0;      // one pool: the value of a token is its key row
      }
      if (c.qk_norm < DN_QKNORM_NONE || c.qk_norm > DN_QKNORM_HEAD) { rc = fail(DN_EINVAL, "layer %d: q / k norm %d unknown", i, c.qk_norm); break; }
      if (c.pool < 0 || (c.pool > 0 && (c.mask_kind != DN_MASK_WINDOW || c.chunk <= 0 || c.kv_from >= 0))) {
        rc = fail(DN_EINVAL, "layer %d: pooled blocks of %d tokens stand behind a sliding window of the layer's own keys", i, c.pool);
        break;
      }
      if (c.qtemp_every < 0 || (c.rot_layout == DN_ROT_HALF && c.dim < c.rot_dims)) { rc = fail(DN_EINVAL, "layer %d: query scale / rotary layout unsupported", i); break; }
      if (c.rot_dims > 0) {
        // frequencies base^(-2j/dims); scaled: dims that turn fast within the original context keep theirs, slow ones are
        // divided by the factor, a linear ramp over the dim index between
        std::vector<float> f(c.rot_dims / 2);
        const double dims = c.rot_dims, base = c.rot_base;
        double lo = 0, hi = 0;
        if (c.yarn_factor > 0.f) {
          auto dim_of = [&](double turns) { return dims * std::log((double)c.yarn_original / (2.0 * M_PI * turns)) / (2.0 * std::log(base)); };
          lo = std::max(std::floor(dim_of(c.yarn_fast)), 0.0);
          hi = std::min(std::ceil(dim_of(c.yarn_slow)), dims - 1.0);
        }
        for (int j = 0; j < c.rot_dims / 2; j++) {
          double fj = std::pow(base, -2.0 * j / dims);
          if (c.yarn_factor > 0.f) {
            const double ramp = std::min(1.0, std::max(0.0, ((double)j - lo) / std::max(hi - lo, 0.001)));
            fj = fj / (double)c.yarn_factor * ramp + fj * (1.0 - ramp);
          }
          f[j] = (float)fj;
        }
        if ((rc = dalloc(&l.inv_freq, f.size() * 4)) != DN_OK) break;
        if (cudaMemcpy(l.inv_freq, f.data(), f.size() * 4, cudaMemcpyHostToDevice) != cudaSuccess) { rc = fail(DN_ECUDA, "inv_freq upload failed"); break; }
      }
      if (c.mixer == DN_MIX_PARALLEL && c.branch_norm && (cfg->streams > 0 || cfg->post_norm)) {
        rc = fail(DN_EINVAL, "layer %d: normed halves of a parallel mixer join the plain residual without a norm after the sublayer", i);
        break;
      }
      if (c.mixer == DN_MIX_PARALLEL && c.r_kind == DN_RIGHT_GDELTA) {
        if (c.r_heads <= 0 || c.r_dim <= 0 || c.r_dim > 1024 || c.r_vdim != c.r_dim || c.rank <= 0 || c.conv > 0 || c.kv_from >= 0) {
          rc = fail(DN_EINVAL, "layer %d: generalized delta rule with heads %d / dim %d / vdim %d / rank %d unsupported", i, c.r_heads, c.r_dim, c.r_vdim, c.rank);
          break;
        }
        l.Rc = l.Rv = c.r_heads * c.r_dim;
        mdq = std::max(mdq, l.Rc);
        mrank = std::max(mrank, c.rank);
        mh = std::max(mh, c.r_heads);
        any_gdelta = true;
      } else if (c.mixer == DN_MIX_PARALLEL) {
        if (c.r_kind != DN_RIGHT_GLA) { rc = fail(DN_EINVAL, "layer %d: right half %d unknown", i, c.r_kind); break; }
        if (c.r_heads <= 0 || c.r_dim <= 0 || c.r_dim > 1024 || c.r_vdim <= 0 || c.rank <= 0 || !(c.tau > 0.f)) {
          rc = fail(DN_EINVAL, "layer %d: linear-attention half heads %d / dim %d / vdim %d / rank %d / tau %g unsupported", i, c.r_heads, c.r_dim, c.r_vdim, c.rank, c.tau);
          break;
        }
        if (c.conv > 0 || c.kv_from >= 0) { rc = fail(DN_EINVAL, "layer %d: a parallel mixer has neither convolutions nor borrowed keys", i); break; }
        l.Rc = c.r_heads * c.r_dim;
        l.Rv = c.r_heads * c.r_vdim;
        mdq = std::max(mdq, l.Rc);
        mrank = std::max(mrank, c.rank);
        mh = std::max(mh, c.r_heads);
      }
    } else if (c.mixer == DN_MIX_LATENT) {
      if (c.kv_rank <= 0 || c.kv_rank > 512 || c.q_rank < 0 || c.rot_part < 0 || c.rot_dims < 0 || c.rot_dims > c.rot_part || (c.rot_dims & 1) ||
          c.kv_heads != 1 || c.conv > 0 || c.kv_from >= 0 || c.sink || c.qk_norm) {
        rc = fail(DN_EINVAL, "layer %d: latent attention with kv_rank %d (1..512) / q_rank %d / rotated part %d of which %d turn unsupported", i,
                  c.kv_rank, c.q_rank, c.rot_part, c.rot_dims);
        break;
      }
      l.Cq = c.heads * (c.dim + c.rot_part);
      l.Ck = c.kv_rank + c.rot_part;       // the cached row: [latent; rotated key part]
      l.Cv = 0;
      l.Co = c.heads * c.vdim;
      l.Cql = c.heads * l.Ck;
      l.Col = c.heads * c.kv_rank;
      mrank = std::max(mrank, c.q_rank);
      m->part_dv = std::max(m->part_dv, (c.kv_rank + 31) / 32 * 32);
      if (c.rot_dims > 0) {
        std::vector<float> f(c.rot_dims / 2);
        for (int j = 0; j < c.rot_dims / 2; j++) f[j] = (float)std::pow((double)c.rot_base, -2.0 * j / (double)c.rot_dims);
        if ((rc = dalloc(&l.inv_freq, f.size() * 4)) != DN_OK) break;
        if (cudaMemcpy(l.inv_freq, f.data(), f.size() * 4, cudaMemcpyHostToDevice) != cudaSuccess) { rc = fail(DN_ECUDA, "inv_freq upload failed"); break; }
      }
    } else if (c.mixer == DN_MIX_DELTA) {
      if (c.dim > 1024) { rc = fail(DN_EINVAL, "layer %d: delta dim %d > 1024", i, c.dim); break; }
      l.Cq = l.Ck = c.kv_heads * c.dim;
      l.Cv = l.Co = c.heads * c.vdim;
      mdq = std::max(mdq, l.Cq);
    } else if (c.mixer == DN_MIX_WKV) {
      if (c.dim > 1024 || c.rank <= 0 || c.conv > 0) { rc = fail(DN_EINVAL, "layer %d: wkv dim %d / rank %d / conv %d unsupported", i, c.dim, c.rank, c.conv); break; }
      l.Cq = l.Ck = c.heads * c.dim;
      l.Cv = l.Co = c.heads * c.vdim;
      mdq = std::max(mdq, l.Cq);
      mrank = std::max(mrank, c.rank);
      any_wkv = true;
    } else {
      rc = fail(DN_EINVAL, "layer %d: mixer %d unknown", i, c.mixer);
      break;
    }
    if (c.mlp_kind == DN_MLP_MOE && c.ff > 0) {
      const int Et = c.experts + (c.router_kind == DN_ROUTER_SCORED ? c.identity : 0);
      if (c.experts <= 0 || c.experts > 4096 || c.top <= 0 || c.top > 16 || c.top > Et || c.shared_ff < 0) {
        rc = fail(DN_EINVAL, "layer %d: %d experts / top %d unsupported (top <= 16, <= experts)", i, c.experts, c.top);
        break;
      }
      if (c.router_kind != DN_ROUTER_TOPK && c.router_kind != DN_ROUTER_SCORED) { rc = fail(DN_EINVAL, "layer %d: router kind %d unknown", i, c.router_kind); break; }
      if (c.expert_act != DN_EXPERT_CGLU && c.expert_act != DN_EXPERT_SWIGLU) { rc = fail(DN_EINVAL, "layer %d: expert activation %d unknown", i, c.expert_act); break; }
      if (c.router_kind == DN_ROUTER_SCORED && (c.identity < 0 || c.groups < 0 || c.groups > 256 ||
                                                (c.groups > 0 && (Et % c.groups || c.groups_keep < 1 || c.groups_keep > c.groups)))) {
        rc = fail(DN_EINVAL, "layer %d: %d + %d experts in %d groups of which %d are kept unsupported", i, c.experts, c.identity, c.groups, c.groups_keep);
        break;
      }
      if ((c.shared_gate || (c.router_kind == DN_ROUTER_SCORED && c.identity > 0)) && !(cfg->post_norm && cfg->streams <= 0)) {
        rc = fail(DN_EINVAL, "layer %d: a gated shared expert and identity experts are joined by the kernels of a norm after the sublayer on the plain residual", i);
        break;
      }
      l.etab_h.assign((size_t)3 * c.experts, nullptr);
      if ((rc = dalloc(&l.etab_d, (size_t)3 * c.experts * sizeof(void*))) != DN_OK) break;
      l.emap_ok.assign((size_t)3 * c.experts, 0);
      if (cfg->dtype == DN_SEQ_BF16 && (rc = dalloc(&l.emaps_d, (size_t)3 * c.experts * sizeof(CUtensorMap))) != DN_OK) break;
      mpairs = std::max(mpairs, c.top);
      meff = std::max(meff, c.ff);
      mexp = std::max(mexp, Et);
      mff = std::max(mff, c.shared_ff);
    } else if (c.mlp_kind != DN_MLP_DENSE && c.ff > 0) {
      rc = fail(DN_EINVAL, "layer %d: feed-forward kind %d unknown", i, c.mlp_kind);
      break;
    } else {
      if (c.ff > 0 && c.ff_act != DN_FF_GEGLU && c.ff_act != DN_FF_RELU2) { rc = fail(DN_EINVAL, "layer %d: feed-forward activation %d unknown", i, c.ff_act); break; }
      mff = std::max(mff, c.ff);
    }
    mq = std::max(mq, l.Cql); mo = std::max(mo, l.Col);
    mq = std::max(mq, std::max(l.Cq, l.Rc)); mk = std::max(mk, std::max(l.Ck, l.Rc)); mv = std::max(mv, std::max(l.Cv, l.Rv));
    mo = std::max(mo, std::max(l.Co, l.Rv));
    mh = std::max(mh, c.heads);
  }
  // the order of layer runs, and every run's own pages and state
  size_t coff = 0, doff = 0;
  if (rc == DN_OK) {
    std::vector<std::pair<int, bool>> order;
    for (int i = 0; i < cfg->n_layers; i++) {
      if (looped && i == cfg->loop_start) {
        for (int t = 0; t < cfg->loop_times; t++)
          for (int j = cfg->loop_start; j < cfg->loop_stop; j++) order.emplace_back(j, j == cfg->loop_start);
        i = cfg->loop_stop - 1;
      } else order.emplace_back(i, false);
    }
    std::vector<int> last_run(cfg->n_layers, -1);
    for (auto& o : order) {
      Run r{o.first, o.second, -1, 0, 0, {0, 0}};
      const SeqLayer& l = m->L[r.layer];
      const dn_seq_layer_cfg& c = l.c;
      if (c.mixer == DN_MIX_ATTENTION || c.mixer == DN_MIX_PARALLEL || c.mixer == DN_MIX_LATENT) {
        if (c.kv_from >= 0) r.kv_index = m->runs[last_run[c.kv_from]].kv_index;
        else {
          r.kv_index = (int)m->kpool.size();
          m->kpool.push_back(nullptr);
          m->vpool.push_back(nullptr);
          m->pkpool.push_back(nullptr);
          m->pvpool.push_back(nullptr);
          if ((rc = dalloc(&m->kpool.back(), (size_t)cfg->pool_pages * PAGE * l.Ck * m->esz)) != DN_OK) break;
          if ((rc = dalloc(&m->vpool.back(), (size_t)cfg->pool_pages * PAGE * l.Cv * m->esz)) != DN_OK) break;
          if (c.pool > 0) {
            const size_t rows = (size_t)cfg->pool_pages * pool_rows(c.pool);
            if ((rc = dalloc(&m->pkpool.back(), rows * l.Ck * m->esz)) != DN_OK) break;
            if ((rc = dalloc(&m->pvpool.back(), rows * l.Cv * m->esz)) != DN_OK) break;
          }
        }
      }
      for (int q = 0; q < 2; q++) {
        r.canon_off[q] = coff;
        if (cfg->canon_taps > 1 && (q == 0 || c.ff > 0)) coff += (size_t)(cfg->canon_taps - 1) * cfg->width;
      }
      r.conv_off = coff;
      if (c.conv > 1) coff += (size_t)(c.conv - 1) * (l.Cq + l.Ck + l.Cv);
      if (c.mixer == DN_MIX_WKV) coff += (size_t)cfg->width;       // the previous token's input row
      r.state_off = doff;
      if (c.mixer == DN_MIX_DELTA || c.mixer == DN_MIX_WKV) doff += (size_t)c.heads * c.dim * c.vdim;
      if (c.mixer == DN_MIX_PARALLEL) doff += (size_t)c.r_heads * c.r_dim * c.r_vdim;
      last_run[r.layer] = (int)m->runs.size();
      m->runs.push_back(r);
    }
  }
  const size_t MB = m->MB, W = cfg->width, e = m->esz;
  m->conv_stride = coff;
  m->delta_stride = doff;
#define DA(p, bytes) if (rc == DN_OK) rc = dalloc(&p, (bytes))
  DA(m->xs, (size_t)m->S1 * MB * W * 4); DA(m->y, MB * W * 4); DA(m->pa, MB * mh * 4); DA(m->pb, MB * mh * 4);
  DA(m->qn, MB * mdq * 4); DA(m->kn, MB * mdq * 4); DA(m->vv, MB * mo * 4); DA(m->od, MB * mo * 4);
  DA(m->beta, MB * mh * 4); DA(m->decay, MB * mh * 4);
  DA(m->y2, MB * W * 4); DA(m->dz, MB * mdq * 4); DA(m->lr, MB * mrank * e);
  DA(m->attn_part, (size_t)AT_SPLIT_ROWS * mh * AT_MAX_SPLITS * (2 + m->part_dv) * 4);
  DA(m->sgate, MB * 4);
  if (looped) { DA(m->x0, MB * W * 4); DA(m->cat, MB * 2 * W * e); }
  if (any_wkv) DA(m->xm, (size_t)SHIFT_MAX * MB * W * e);
  if (cfg->canon_taps > 0) DA(m->hn, MB * W * e);
  if (any_gdelta) { DA(m->un, MB * mdq * 4); DA(m->aun, MB * mdq * 4); }
  if (mpairs > 0) {
    const size_t P = MB * mpairs;
    m->max_tiles = (int)(P / MOE_ROWS) + mexp + 1;
    DA(m->ridx, P * 4); DA(m->rpos, P * 4); DA(m->rtok, P * 4); DA(m->rwt, P * 4); DA(m->tiles, ((size_t)3 * m->max_tiles + 4) * 4);
    DA(m->eact, P * meff * e); DA(m->eo, P * W * 4);
    if (cfg->dtype == DN_SEQ_BF16) DA(m->xg, P * W * e);
  }
  DA(m->h, MB * W * e); DA(m->uq, MB * mq * e); DA(m->uk, MB * mk * e); DA(m->uv, MB * mv * e); DA(m->qb, MB * mq * e);
  DA(m->mo, MB * mo * e); DA(m->gt, MB * mo * e); DA(m->act, MB * mff * e);
  DA(m->conv_state, (size_t)cfg->max_seqs * coff * e); DA(m->delta_state, (size_t)cfg->max_seqs * doff * 4);
  m->stage_ints = 5 * MB + 3 * (size_t)(cfg->max_seqs + 1) + MB;
  DA(m->stage_d, m->stage_ints * 4); DA(m->bt_d, (size_t)cfg->max_seqs * m->max_pages * 4); DA(m->tc_err, 16);
  DA(m->lg_buf, (size_t)8 * cfg->vocab * 4);
#undef DA
  if (rc == DN_OK && cudaMemset(m->tc_err, 0, 16) != cudaSuccess) rc = fail(DN_ECUDA, "memset failed");
  if (rc == DN_OK && cfg->dtype == DN_SEQ_BF16) {
    make_xmaps(&m->x_h, m->h, m->MB, cfg->width);
    for (auto& l : m->L) {
      make_xmaps(&l.x_mo, m->mo, m->MB, l.Co);
      if (l.Rv > 0) make_xmaps(&l.x_mo_r, m->mo, m->MB, l.Rv);
      if (l.c.rank > 0) make_xmaps(&l.x_lr, m->lr, m->MB, l.c.rank);
      if (l.c.mixer == DN_MIX_LATENT && l.c.q_rank > 0) make_xmaps(&l.x_lr, m->lr, m->MB, l.c.q_rank);
      const int fa = l.c.mlp_kind == DN_MLP_MOE ? l.c.shared_ff : l.c.ff;
      if (fa > 0) make_xmaps(&l.x_act, m->act, m->MB, fa);
    }
    if (m->xg) {
      m->x_xg_ok = make_tmap(&m->x_xg[0], m->xg, m->MB * mpairs, cfg->width, 64) && make_tmap(&m->x_xg[1], m->xg, m->MB * mpairs, cfg->width, 128);
      for (auto& l : m->L)
        if (l.c.mlp_kind == DN_MLP_MOE && l.c.ff > 0)
          l.x_eact_ok = make_tmap(&l.x_eact[0], m->eact, m->MB * l.c.top, l.c.ff, 64) && make_tmap(&l.x_eact[1], m->eact, m->MB * l.c.top, l.c.ff, 128);
    }
    if (m->cat) make_xmaps(&m->x_cat, m->cat, m->MB, 2 * cfg->width);
    if (m->xm) for (int i = 0; i < SHIFT_MAX; i++) make_xmaps(&m->x_xm[i], (char*)m->xm + (size_t)i * MB * W * e, m->MB, cfg->width);
  }
  if (rc == DN_OK && cudaHostAlloc((void**)&m->stage_h, m->stage_ints * 4, cudaHostAllocPortable) != cudaSuccess) rc = fail(DN_ENOMEM, "pinned staging failed");
  if (rc == DN_OK && cudaHostAlloc((void**)&m->bt_h, (size_t)cfg->max_seqs * m->max_pages * 4, cudaHostAllocPortable) != cudaSuccess) rc = fail(DN_ENOMEM, "pinned block table failed");
  if (rc == DN_OK && cudaEventCreateWithFlags(&m->staged, cudaEventDisableTiming) != cudaSuccess) rc = fail(DN_ECUDA, "event creation failed");
  if (rc != DN_OK) { dn_seq_model_destroy(m); return rc; }
  for (int p = cfg->pool_pages - 1; p >= 0; p--) m->free_pages.push_back(p);
  for (int s = cfg->max_seqs - 1; s >= 0; s--) m->free_slots.push_back(s);
  m->pages.resize(cfg->max_seqs);
  m->length.assign(cfg->max_seqs, -1);
  m->last_tok.assign(cfg->max_seqs, -1);
  *out = m;
  return DN_OK;
}

extern "C" int dn_seq_bind(dn_seq_model* m, int layer, int which, const void* p) {
  if (!m) return fail(DN_EINVAL, "null model");
  const bool b16 = m->cfg.dtype == DN_SEQ_BF16;
  for (auto& g : m->graphs) cudaGraphExecDestroy(g.second.first);     // captured steps hold the old pointers
  m->graphs.clear();
  if (layer < 0) {
    if (which == DN_SQ_EMBED) m->embed = p;
    else if (which == DN_SQ_FINAL_NORM) m->final_norm = p;
    else if (which == DN_SQ_HEAD) {
      m->head = p;
      m->tm_head_ok = b16 && make_tmap(&m->tm_head, p, m->cfg.vocab, m->cfg.width, dn::TC_BM);
    } else if (which > DN_SQ_HEAD && which <= DN_SQ_BIGRAM) {
      m->mw[which - DN_SQ_EMBED] = p;
      if (which == DN_SQ_LOOP_IN) m->tm_loop_ok = b16 && make_tmap(&m->tm_loop_in, p, m->cfg.width, 2 * m->cfg.width, dn::TC_BM);
    } else return fail(DN_EINVAL, "tensor %d is not a model tensor", which);
    return DN_OK;
  }
  if (layer >= (int)m->L.size() || which < 0 || which >= DN_SQ_COUNT) return fail(DN_EINVAL, "layer %d / tensor %d out of range", layer, which);
  SeqLayer& l = m->L[layer];
  l.w[which] = p;
  int rows = 0, cols = m->cfg.width;
  switch (which) {
    case DN_SQ_Q: rows = l.Cq; if (l.c.mixer == DN_MIX_LATENT && l.c.q_rank > 0) cols = l.c.q_rank; break;
    case DN_SQ_DQ: rows = l.c.q_rank; break;
    case DN_SQ_DKV: rows = l.Ck; break;
    case DN_SQ_K: rows = l.Ck; break;
    case DN_SQ_V: rows = l.Cv; break;
    case DN_SQ_G: rows = l.Co; break;
    case DN_SQ_A: case DN_SQ_B: rows = l.c.heads; break;
    case DN_SQ_GATE: case DN_SQ_UP: rows = l.c.ff; break;
    case DN_SQ_O: rows = m->cfg.width; cols = l.Co; break;
    case DN_SQ_DOWN: rows = m->cfg.width; cols = l.c.ff; break;
    case DN_SQ_HEAD_GATE: rows = l.c.heads; break;
    case DN_SQ_R_Q: case DN_SQ_R_K: case DN_SQ_R_A: rows = l.Rc; break;
    case DN_SQ_R_V: case DN_SQ_R_G: rows = l.Rv; break;
    case DN_SQ_R_O: rows = m->cfg.width; cols = l.Rv; break;
    case DN_SQ_DECAY1: rows = l.c.rank; break;
    case DN_SQ_DECAY2: rows = l.c.mixer == DN_MIX_PARALLEL ? l.Rc : l.Cq; cols = l.c.rank; break;
    case DN_SQ_SH_GATE: case DN_SQ_SH_UP: rows = l.c.shared_ff; break;
    case DN_SQ_SH_DOWN: rows = m->cfg.width; cols = l.c.shared_ff; break;
    default: break;
  }
  if (l.c.mlp_kind == DN_MLP_MOE && (which == DN_SQ_GATE || which == DN_SQ_UP || which == DN_SQ_DOWN))
    return fail(DN_EINVAL, "layer %d: the matrices of routed experts are bound with dn_seq_bind_expert", layer);
  l.tm_ok[which] = b16 && rows > 0 && make_tmap(&l.tm[which], p, rows, cols, dn::TC_BM);
  return DN_OK;
}

extern "C" int dn_seq_bind_expert(dn_seq_model* m, int layer, int expert, int which, const void* p) {
  if (!m) return fail(DN_EINVAL, "null model");
  if (layer < 0 || layer >= (int)m->L.size()) return fail(DN_EINVAL, "layer %d out of range", layer);
  SeqLayer& l = m->L[layer];
  if (l.c.mlp_kind != DN_MLP_MOE || l.c.ff <= 0) return fail(DN_EINVAL, "layer %d has no routed experts", layer);
  if (expert < 0 || expert >= l.c.experts || which < DN_SQ_E_GATE || which > DN_SQ_E_DOWN) return fail(DN_EINVAL, "expert %d / matrix %d out of range", expert, which);
  for (auto& g : m->graphs) cudaGraphExecDestroy(g.second.first);
  m->graphs.clear();
  const size_t at = (size_t)which * l.c.experts + expert;
  l.etab_h[at] = p;
  CK(cudaMemcpy((void*)(l.etab_d + at), &p, sizeof(void*), cudaMemcpyHostToDevice));
  if (l.emaps_d) {
    CUtensorMap tm;
    const bool down = which == DN_SQ_E_DOWN;
    l.emap_ok[at] = make_tmap(&tm, p, down ? m->cfg.width : l.c.ff, down ? l.c.ff : m->cfg.width, dn::TC_BM) ? 1 : 0;
    if (l.emap_ok[at]) CK(cudaMemcpy(l.emaps_d + at, &tm, sizeof(tm), cudaMemcpyHostToDevice));
  }
  return DN_OK;
}
extern "C" int dn_seq_layer_runs(dn_seq_model* m) { return m ? (int)m->runs.size() : DN_EINVAL; }

extern "C" int dn_seq_open(dn_seq_model* m, dn_seq_stream s, int* slot_out) {
  if (!m || !slot_out) return fail(DN_EINVAL, "null argument");
  if (m->free_slots.empty()) return fail(DN_ENOSPC, "all %d state slots are in use", m->cfg.max_seqs);
  const int slot = m->free_slots.back();
  // the slot's recurrent state and carried conv inputs start at zero, behind whatever still reads the slot on s
  if (m->conv_stride) CK(cudaMemsetAsync((char*)m->conv_state + (size_t)slot * m->conv_stride * m->esz, 0, m->conv_stride * m->esz, (cudaStream_t)s));
  if (m->delta_stride) CK(cudaMemsetAsync(m->delta_state + (size_t)slot * m->delta_stride, 0, m->delta_stride * 4, (cudaStream_t)s));
  m->free_slots.pop_back();
  m->length[slot] = 0;
  m->last_tok[slot] = -1;
  m->pages[slot].clear();
  *slot_out = slot;
  return DN_OK;
}

extern "C" int dn_seq_close(dn_seq_model* m, int slot) {
  if (!m || slot < 0 || slot >= m->cfg.max_seqs || m->length[slot] < 0) return fail(DN_EINVAL, "slot %d is not open", slot);
  for (auto it = m->pages[slot].rbegin(); it != m->pages[slot].rend(); ++it) m->free_pages.push_back(*it);
  m->pages[slot].clear();
  m->length[slot] = -1;
  m->free_slots.push_back(slot);
  return DN_OK;
}

extern "C" int dn_seq_length(dn_seq_model* m, int slot) {
  if (!m || slot < 0 || slot >= m->cfg.max_seqs) return DN_EINVAL;
  return m->length[slot];
}
extern "C" int dn_seq_check(dn_seq_model* m, dn_seq_stream s) {
  if (!m) return fail(DN_EINVAL, "null model");
  unsigned int e = 0;
  CK(cudaMemcpyAsync(&e, m->tc_err, 4, cudaMemcpyDeviceToHost, (cudaStream_t)s));
  CK(cudaStreamSynchronize((cudaStream_t)s));
  if (e) return fail(-62, "a bounded wait inside a GEMM kernel ran out (code %u): results of this model are invalid", e);
  return DN_OK;
}
extern "C" int dn_seq_profile(dn_seq_model* m, int on) {
  if (!m) return fail(DN_EINVAL, "null model");
  m->prof_on = on != 0;
  return DN_OK;
}
extern "C" int dn_seq_profile_read(dn_seq_model* m, double* ms_out, int reset) {
  if (!m || !ms_out) return fail(DN_EINVAL, "bad argument");
  CK(cudaDeviceSynchronize());
  for (size_t i = 0; i + 1 < m->prof_marks.size(); i++) {
    float ms = 0.f;
    // a step's last mark closes it: the gap to the next step's first mark is host time, not a phase
    if (m->prof_marks[i].first != DN_SEQ_PH_OTHER || m->prof_marks[i + 1].first != DN_SEQ_PH_EMBED) {
      CK(cudaEventElapsedTime(&ms, m->prof_marks[i].second, m->prof_marks[i + 1].second));
      m->prof_ms[m->prof_marks[i].first] += ms;
    }
  }
  for (auto& pm : m->prof_marks) m->prof_pool.push_back(pm.second);
  m->prof_marks.clear();
  for (int i = 0; i < DN_SEQ_PH_COUNT; i++) ms_out[i] = m->prof_ms[i];
  if (reset) for (int i = 0; i < DN_SEQ_PH_COUNT; i++) m->prof_ms[i] = 0;
  return DN_OK;
}
extern "C" int dn_seq_free_pages(dn_seq_model* m) { return m ? (int)m->free_pages.size() : DN_EINVAL; }
extern "C" int dn_seq_free_slots(dn_seq_model* m) { return m ? (int)m->free_slots.size() : DN_EINVAL; }

// ---------------------------------------------------------------------------------------------------------------
template <int BN, int EPI, int STAGES>
static cudaError_t launch_tc(const CUtensorMap& w, const CUtensorMap& w2, const CUtensorMap& x, const dn::TcParams& p, cudaStream_t s) {
  constexpr int NA = dn::epi_two_weights(EPI) ? 2 : 1;
  constexpr size_t smem = (size_t)STAGES * (NA * dn::TC_BM * dn::TC_BK * 2 + BN * dn::TC_BK * 2) + 1024 + 256;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(dn::k_gemm_tc<BN, EPI, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    attr = true;
  }
  const int tiles = ((p.N + dn::TC_BM - 1) / dn::TC_BM) * ((p.T + BN - 1) / BN);
  g_launches++;
  dn::k_gemm_tc<BN, EPI, STAGES><<<tiles < g_sms ? tiles : g_sms, dn::TC_THREADS, smem, s>>>(w, w2, x, p);
  return cudaGetLastError();
}
// token-tile width: the widest that still gives about one CTA per SM
template <int EPI>
static cudaError_t gemm_tc(const CUtensorMap& w, const CUtensorMap& w2, const XMaps& x, const dn::TcParams& p, cudaStream_t s) {
  constexpr bool two = dn::epi_two_weights(EPI);
  const int n_tiles = (p.N + dn::TC_BM - 1) / dn::TC_BM;
  auto tiles = [&](int bn) { return n_tiles * ((p.T + bn - 1) / bn); };
  if (p.T > 64 && tiles(128) >= 100) return launch_tc<128, EPI, (two ? 4 : 6)>(w, w2, x.m[2], p, s);
  if (p.T > 32 && (tiles(64) >= 100 || tiles(64) * 2 > tiles(32))) return launch_tc<64, EPI, (two ? 5 : 8)>(w, w2, x.m[1], p, s);
  return launch_tc<32, EPI, (two ? 5 : 8)>(w, w2, x.m[0], p, s);
}

// One product Y[N, O] = X[N, K] W[O, K]^T (act: an ACT_* epilogue, the two-operand ones on X W^T and X W2^T).  bf16 batches of 16 tokens and more run on
// the tcgen05 GEMM when the operands have TMA descriptors; a few rows (decode) on the weight-streaming row kernel;
// everything else, and all of fp32, on the CUDA-core tiles.
struct LinMaps { const CUtensorMap* w; const CUtensorMap* w2; const XMaps* x; };
template <class T>
static cudaError_t linear(dn_seq_model* m, cudaStream_t s, const T* X, const void* W, const void* W2, void* Y, int N, int O, int K, bool out32,
                          int act, LinMaps tm = LinMaps{nullptr, nullptr, nullptr}, float alim = 0.f, const void* bias = nullptr) {
  // (a weight of fewer than 128 rows fills part of a tile: still far ahead of the CUDA-core tiles once K is in the thousands)
  if (std::is_same<T, bf16>::value && N >= 16 && O >= 16 && tm.w && tm.x && tm.x->ok && (!bias || act == ACT_RELU2 || (act == ACT_NONE && out32)) &&
      (act == ACT_NONE || act == ACT_TANH || act == ACT_RELU2 || (act_two(act) && tm.w2))) {
    dn::TcParams p;
    memset(&p, 0, sizeof(p));
    p.T = N; p.N = O; p.K = K; p.ldy = O; p.Y = (dn::bf16*)Y; p.err = m->tc_err; p.limit = alim; p.bias = (const dn::bf16*)bias;
    if (act == ACT_CGLU) return gemm_tc<dn::EPI_CGLU>(*tm.w, *tm.w2, *tm.x, p, s);
    if (act == ACT_SWIGLU) return gemm_tc<dn::EPI_SGLU>(*tm.w, *tm.w2, *tm.x, p, s);
    if (act == ACT_RELU2) return gemm_tc<dn::EPI_RELU2>(*tm.w, *tm.w, *tm.x, p, s);
    if (act == ACT_TANH) return gemm_tc<dn::EPI_TANH>(*tm.w, *tm.w, *tm.x, p, s);
    if (act) return gemm_tc<dn::EPI_GEGLU>(*tm.w, *tm.w2, *tm.x, p, s);
    if (out32) return gemm_tc<dn::EPI_STORE_F32>(*tm.w, *tm.w, *tm.x, p, s);
    return gemm_tc<dn::EPI_STORE>(*tm.w, *tm.w, *tm.x, p, s);
  }
  if (N <= 8) {
    dim3 grid((O + 7) / 8);
    if (out32) return launch(k_linear_rows<T, true>, grid, dim3(256), 0, s, X, (const T*)W, (const T*)W2, Y, N, O, K, act, alim, (const T*)bias);
    return launch(k_linear_rows<T, false>, grid, dim3(256), 0, s, X, (const T*)W, (const T*)W2, Y, N, O, K, act, alim, (const T*)bias);
  }
  dim3 grid((O + 63) / 64, (N + 63) / 64);
  if (out32) return launch(k_linear<T, true>, grid, dim3(256), 0, s, X, (const T*)W, (const T*)W2, Y, N, O, K, act, alim, (const T*)bias);
  return launch(k_linear<T, false>, grid, dim3(256), 0, s, X, (const T*)W, (const T*)W2, Y, N, O, K, act, alim, (const T*)bias);
}

// Attention of a step: bf16 steps that bring a prompt portion (an entry of 16 tokens or more) run on the MMA tiles when
// the head sizes fit its templates; decode-only steps, odd head sizes and fp32 on the one-warp-per-(token, head) kernel.
template <class T>
static bool attn_tiles_ok(const dn_seq_layer_cfg& lc, const Batch& b) {
  return std::is_same<T, bf16>::value && b.max_len >= 16 && lc.dim % 8 == 0 && lc.vdim % 8 == 0 && lc.dim <= 128 && lc.vdim <= 128;
}
template <int DKP, int DVP>
static cudaError_t attn_tiles_launch(cudaStream_t s, const Batch& b, const bf16* q, const bf16* kp, const bf16* vp, const dn_seq_layer_cfg& lc,
                                     const AttnExtra& ex, bf16* out) {
  constexpr size_t smem = ((size_t)2 * AT_ROWS * (DKP + 8) + (size_t)AT_ROWS * (DVP + 8)) * 2;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(k_attn_tiles<DKP, DVP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    attr = true;
  }
  g_launches++;
  k_attn_tiles<DKP, DVP><<<dim3(b.row_tiles, lc.heads), 128, smem, s>>>(b, q, kp, vp, lc.heads, lc.kv_heads, lc.dim, lc.vdim, lc.chunk, lc.scale, ex, out);
  return cudaGetLastError();
}
static cudaError_t attn_tiles(cudaStream_t s, const Batch& b, const bf16* q, const bf16* kp, const bf16* vp, const dn_seq_layer_cfg& lc,
                              const AttnExtra& ex, bf16* out) {
  const int kq = lc.dim <= 32 ? 0 : lc.dim <= 64 ? 1 : 2, vq = lc.vdim <= 32 ? 0 : lc.vdim <= 64 ? 1 : 2;
#define AT(a, c, A, Cc) if (kq == a && vq == c) return attn_tiles_launch<A, Cc>(s, b, q, kp, vp, lc, ex, out);
  AT(0, 0, 32, 32) AT(0, 1, 32, 64) AT(0, 2, 32, 128) AT(1, 0, 64, 32) AT(1, 1, 64, 64) AT(1, 2, 64, 128)
  AT(2, 0, 128, 32) AT(2, 1, 128, 64) AT(2, 2, 128, 128)
#undef AT
  return cudaErrorInvalidValue;
}

// latent attention of a step that brings a prompt portion, bf16: the MMA tiles over the cached rows (R + rot numbers a key,
// the first R the value) when the rows start on 16-byte boundaries
static bool latent_tiles_ok(const Batch& b, int Ck, int R) {
  const int DKP = (Ck + 15) / 16 * 16, DVH = R <= 128 ? 64 : R <= 256 ? 128 : 256, LD = std::max(DKP, 2 * DVH) + 8;
  return Ck % 8 == 0 && R % 2 == 0 && R <= 512 && (size_t)3 * 64 * LD * 2 <= g_max_smem;      // three tiles must fit the shared memory
}
template <int DVH, int MODE>
static cudaError_t latent_tiles_launch(cudaStream_t s, const Batch& b, const bf16* q, const bf16* pool, int H, int Ck, int R, int chunk, float scale,
                                       const AttnExtra& ex, bf16* out, float* part, int part_ld, int zmax) {
  const int DKP = (Ck + 15) / 16 * 16, LD = std::max(DKP, 2 * DVH) + 8;
  const size_t smem = (size_t)3 * 64 * LD * 2;      // the query tile and two key tiles
  static size_t attr = 0;
  if (smem > attr) {
    cudaError_t e = cudaFuncSetAttribute(k_latent_tiles<DVH, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    attr = smem;
  }
  g_launches++;
  const dim3 grid = MODE ? dim3(b.N, (H + 63) / 64, zmax) : dim3(b.row_tiles, H);
  k_latent_tiles<DVH, MODE><<<grid, 256, smem, s>>>(b, q, pool, H, Ck, R, DKP, LD, chunk, scale, ex, out, part, part_ld);
  return cudaGetLastError();
}
// prompt portions: a block per (64 rows, head); decode steps (every entry one token): a block per (token, 64 heads, split) + the merge.
// The partials' buffer holds AT_SPLIT_ROWS x AT_MAX_SPLITS rows per head: up to 8 tokens are split 32 ways, more 16 ways.
static cudaError_t latent_tiles(cudaStream_t s, const Batch& b, const bf16* q, const bf16* pool, int H, int Ck, int R, int chunk, float scale,
                                const AttnExtra& ex, bf16* out, float* part, int part_ld) {
  const bool dec = b.max_len == 1 && b.N <= AT_SPLIT_ROWS;
  const int zmax = b.N <= 8 ? 32 : AT_MAX_SPLITS;
  const int mode = !dec ? 0 : H <= 16 ? 2 : 1;
  cudaError_t e;
#define LT(D) (mode == 0 ? latent_tiles_launch<D, 0>(s, b, q, pool, H, Ck, R, chunk, scale, ex, out, part, part_ld, zmax) \
             : mode == 1 ? latent_tiles_launch<D, 1>(s, b, q, pool, H, Ck, R, chunk, scale, ex, out, part, part_ld, zmax) \
                         : latent_tiles_launch<D, 2>(s, b, q, pool, H, Ck, R, chunk, scale, ex, out, part, part_ld, zmax))
  if (R <= 128) e = LT(64);
  else if (R <= 256) e = LT(128);
  else e = LT(256);
#undef LT
  if (e != cudaSuccess || !dec) return e;
  g_launches++;
  k_latent_merge<<<dim3(b.N, H), 128, 0, s>>>(b, H, R, chunk, zmax, ex, part, part_ld, out);
  return cudaGetLastError();
}

// phase boundary: the time from this mark to the next one is booked on `phase`
static cudaError_t mark(dn_seq_model* m, int phase, cudaStream_t s) {
  if (!m->prof_on) return cudaSuccess;
  cudaEvent_t ev;
  if (!m->prof_pool.empty()) { ev = m->prof_pool.back(); m->prof_pool.pop_back(); }
  else { cudaError_t e = cudaEventCreate(&ev); if (e != cudaSuccess) return e; }
  m->prof_marks.emplace_back(phase, ev);
  return cudaEventRecord(ev, s);
}

// one launch of the tcgen05 GEMM over all experts of a layer (token tiles of MOE_ROWS rows from the plan)
template <int EPI, int BN>
static cudaError_t gemm_tc_grouped(const CUtensorMap& x, const dn::TcParams& p, cudaStream_t s) {
  constexpr int NA = dn::epi_two_weights(EPI) ? 2 : 1;
  constexpr int STAGES = BN == 128 ? (NA == 2 ? 4 : 6) : (NA == 2 ? 5 : 8);
  constexpr size_t smem = (size_t)STAGES * (NA * dn::TC_BM * dn::TC_BK * 2 + BN * dn::TC_BK * 2) + 1024 + 256;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(dn::k_gemm_tc<BN, EPI, STAGES, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    attr = true;
  }
  g_launches++;
  dn::k_gemm_tc<BN, EPI, STAGES, true><<<g_sms, dn::TC_THREADS, smem, s>>>(x, x, x, p);
  return cudaGetLastError();
}

// the expert products of a routed feed-forward: h [N, W] -> m->y [N, W] (routed sum), m->y2 (shared expert, if any);
// fused: the sum of both goes through the norm after the sublayer into the plain residual in the combining kernel
// combine = false: the caller's joining kernel adds the pairs itself (k_rms_join)
template <class T>
static int moe_ff(dn_seq_model* m, SeqLayer& l, int N, bool fused, NextNorm<T> nx, cudaStream_t s, bool combine = true) {
  const dn_seq_layer_cfg& lc = l.c;
  const bool scored = lc.router_kind == DN_ROUTER_SCORED;
  const int W = m->cfg.width, E = lc.experts, Et = E + (scored ? lc.identity : 0), top = lc.top, P = N * top;
  const int eact = lc.expert_act == DN_EXPERT_SWIGLU ? ACT_SWIGLU : ACT_CGLU;
  auto w = [&](int i) { return (const T*)l.w[i]; };
  auto wm = [&](int i) { return l.tm_ok[i] ? &l.tm[i] : (const CUtensorMap*)nullptr; };
  CK(mark(m, DN_SEQ_PH_ROUTER, s));
  if (scored)
    CK(launch(k_router_scored<T>, dim3(N), dim3(32 * std::min(32, std::max(4, Et + 1))), (size_t)2 * Et * 4, s, (const T*)m->h, w(DN_SQ_ROUTER), w(DN_SQ_ROUTER_CORR),
              W, Et, top, lc.groups, lc.groups_keep, lc.router_scale, lc.shared_gate ? w(DN_SQ_SH_SG) : (const T*)nullptr, m->ridx, m->rwt, m->rpos, m->sgate));
  else
    CK(launch(k_router<T>, dim3(N), dim3(32 * std::min(32, std::max(4, E))), (size_t)E * 4, s, (const T*)m->h, w(DN_SQ_ROUTER), w(DN_SQ_ROUTER_B), W, E, top, m->ridx, m->rwt, m->rpos));
  const bool few = N <= 8;
  if (few) {      // the shared expert's rows ride in the same two launches
    SharedExpert sh{l.w[DN_SQ_SH_GATE], l.w[DN_SQ_SH_UP], l.w[DN_SQ_SH_DOWN], lc.shared_ff, lc.shared_limit, m->act, m->y2};
    const int rows = P + (lc.shared_ff > 0 ? N : 0);
    CK(mark(m, DN_SEQ_PH_MOE_UP, s));
    CK(launch(k_moe_rows<T, true>, dim3((std::max(lc.ff, lc.shared_ff) + 7) / 8, rows), dim3(256), 0, s, (const T*)m->h, (const void* const*)l.etab_d, E,
              (const int32_t*)m->ridx, top, m->eact, lc.ff, W, lc.limit, P, (const T*)m->h, sh, eact));
    CK(mark(m, DN_SEQ_PH_MOE_DOWN, s));
    CK(launch(k_moe_rows<T, false>, dim3((W + 7) / 8, rows), dim3(256), 0, s, (const T*)m->eact, (const void* const*)l.etab_d, E, (const int32_t*)m->ridx, top,
              m->eo, W, lc.ff, 0.f, P, (const T*)m->h, sh, eact));
  } else {
    MoePlan pl{m->rpos, m->rtok, m->tiles, m->tiles + m->max_tiles, m->tiles + 2 * m->max_tiles, m->tiles + 3 * m->max_tiles};
    const int mt = std::min(m->max_tiles, P / MOE_ROWS + E + 1);
    bool tc = std::is_same<T, bf16>::value && m->x_xg_ok && l.x_eact_ok && l.emaps_d && lc.ff >= 32 && W >= 32;
    for (char ok : l.emap_ok) tc = tc && ok;
    // rows of a token tile: 128 (the tensor cores read the weight tile once for twice the tokens) when an expert gets
    // two such tiles on average, else 64 (less padding); the CUDA-core tiles are 64 rows
    const int tile_rows = tc && P / E >= 256 ? 128 : MOE_ROWS;
    CK(launch(k_moe_plan, dim3(1), dim3(1024), (size_t)(2 * Et + 1) * 4, s, (const int32_t*)m->ridx, P, top, Et, tile_rows, pl, E));
    if (tc) {     // bf16 with TMA-able shapes: every expert's tiles in one launch of the tcgen05 GEMM
      CK(launch(k_moe_gather<T>, dim3(P), dim3(128), 0, s, (const T*)m->h, (const int32_t*)m->rtok, W, (T*)m->xg));
      dn::TcParams p;
      memset(&p, 0, sizeof(p));
      p.err = m->tc_err; p.limit = lc.limit;
      p.g_tile_e = pl.tile_e; p.g_tile_r0 = pl.tile_r0; p.g_tile_rows = pl.tile_rows; p.g_ntiles = pl.n_tiles;
      CK(mark(m, DN_SEQ_PH_MOE_UP, s));
      p.T = P; p.N = lc.ff; p.K = W; p.ldy = lc.ff; p.Y = (dn::bf16*)m->eact; p.g_mapW = l.emaps_d; p.g_mapW2 = l.emaps_d + E;
      if (eact == ACT_SWIGLU) {
        if (tile_rows == 128) CK(gemm_tc_grouped<dn::EPI_SGLU, 128>(m->x_xg[1], p, s));
        else CK(gemm_tc_grouped<dn::EPI_SGLU, 64>(m->x_xg[0], p, s));
      } else if (tile_rows == 128) CK(gemm_tc_grouped<dn::EPI_CGLU, 128>(m->x_xg[1], p, s));
      else CK(gemm_tc_grouped<dn::EPI_CGLU, 64>(m->x_xg[0], p, s));
      CK(mark(m, DN_SEQ_PH_MOE_DOWN, s));
      p.N = W; p.K = lc.ff; p.ldy = W; p.Y = (dn::bf16*)m->eo; p.g_mapW = l.emaps_d + 2 * E; p.g_mapW2 = l.emaps_d + 2 * E;
      if (tile_rows == 128) CK(gemm_tc_grouped<dn::EPI_STORE_F32, 128>(l.x_eact[1], p, s));
      else CK(gemm_tc_grouped<dn::EPI_STORE_F32, 64>(l.x_eact[0], p, s));
    } else {
      CK(mark(m, DN_SEQ_PH_MOE_UP, s));
      CK(launch(k_moe_tiles<T, true>, dim3((lc.ff + 63) / 64, mt), dim3(256), 0, s, (const T*)m->h, (const void* const*)l.etab_d, E, pl, m->eact, lc.ff, W, lc.limit, eact));
      CK(mark(m, DN_SEQ_PH_MOE_DOWN, s));
      CK(launch(k_moe_tiles<T, false>, dim3((W + 63) / 64, mt), dim3(256), 0, s, (const T*)m->eact, (const void* const*)l.etab_d, E, pl, m->eo, W, lc.ff, 0.f, eact));
    }
  }
  if (lc.shared_ff > 0 && !few) {
    CK(mark(m, DN_SEQ_PH_FF_UP, s));
    CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_SH_GATE], l.w[DN_SQ_SH_UP], m->act, N, lc.shared_ff, W, false, eact,
                 LinMaps{wm(DN_SQ_SH_GATE), wm(DN_SQ_SH_UP), &m->x_h}, lc.shared_limit));
    CK(mark(m, DN_SEQ_PH_FF_DOWN, s));
    CK(linear<T>(m, s, (const T*)m->act, l.w[DN_SQ_SH_DOWN], nullptr, m->y2, N, W, lc.shared_ff, true, 0, LinMaps{wm(DN_SQ_SH_DOWN), nullptr, &l.x_act}));
  }
  CK(mark(m, DN_SEQ_PH_WRITE_BACK, s));
  if (!combine) return DN_OK;
  CK(launch(k_moe_combine<T>, dim3((unsigned)(((size_t)N * W + 255) / 256)), dim3(256), 0, s, (const float*)m->eo, (const float*)m->rwt, (const int32_t*)m->rpos, N, W, top,
            m->y, fused ? m->xs : (float*)nullptr, lc.shared_ff > 0 ? (const float*)m->y2 : (const float*)nullptr, w(DN_SQ_POST2), w(DN_SQ_POST2_B), w(DN_SQ_POST2_ALPHA), nx,
            scored ? (const int32_t*)m->ridx : (const int32_t*)nullptr, E, (const T*)m->h, lc.shared_gate ? (const float*)m->sgate : (const float*)nullptr));
  return DN_OK;
}

// rows a lane (R) and lanes a column (P) of the recurrences: the smallest P R >= dk of this table
static void recur_shape(int dk, int* R, int* P) {
  static const int RP[8][3] = {{8, 8, 1}, {16, 8, 2}, {32, 8, 4}, {64, 8, 8}, {128, 16, 8}, {256, 16, 16}, {512, 16, 32}, {1024, 32, 32}};
  *R = 32; *P = 32;
  for (int i = 7; i >= 0; i--) if (dk <= RP[i][0]) { *R = RP[i][1]; *P = RP[i][2]; }
}
// a decayed outer-product recurrence over the step's entries: inputs m->qn / kn / vv / dz (fp32), output m->od
static int decay_rule(dn_seq_model* m, const Batch& b, int mode, int H, int dk, int dv, const void* bonus, float* st, cudaStream_t s) {
  int R, P;
  recur_shape(dk, &R, &P);
  // columns a block: 16 where that still fills whole warps (twice the blocks, half the shared-memory reads a block and token)
  const int cols = P >= 2 ? 16 : 32;
  dim3 grid(b.E * H, (dv + cols - 1) / cols);
  const int per = 3 * P * (R + 4) + cols;
  int TB = std::max(1, std::min(16, 5800 / per));      // two tiles within ~46 KB of shared memory
  if (TB >= 8) TB &= ~7;      // whole groups of the kernel's token batches
  else if (TB >= 4) TB = 4;
  const size_t dsm = (size_t)2 * TB * per * 4;
#define DR(Rv, Pv, Cv_) if (R == Rv && P == Pv) CK(launch(k_decay_rule<Rv, Pv, Cv_>, grid, dim3(Cv_ * Pv), dsm, s, mode, b, H, dk, dv, TB, (const float*)m->qn, \
                         (const float*)m->kn, (const float*)m->vv, (const float*)m->dz, bonus, m->esz == 4 ? 1 : 0, st, m->delta_stride, m->od))
  DR(8, 1, 32); DR(8, 2, 16); DR(8, 4, 16); DR(8, 8, 16); DR(16, 8, 16); DR(16, 16, 16); DR(16, 32, 16); DR(32, 32, 16);
#undef DR
  return DN_OK;
}

template <class T>
static int step_T(dn_seq_model* m, const Batch& b, int n_want, const int32_t* want_dev, float* logits, float* trace, cudaStream_t s) {
  const dn_seq_cfg& c = m->cfg;
  const int N = b.N, W = c.width, S = c.streams, S1 = m->S1;
  const size_t NW = (size_t)N * W;
  const size_t nsm = ((size_t)W + 40) * 4;
  const int ew = (int)((NW + 255) / 256), ew4 = (int)((NW / 4 + 255) / 256);
  const dim3 nthr(W >= 4096 ? 512 : W >= 2048 ? 256 : 128);     // threads of a norm block: a function of the width only
  const bool dyt = c.norm_kind == DN_NORM_DYT;
  const int lnorm = c.norm_kind == DN_NORM_LAYER ? 1 : 0;
  const int taps = c.canon_taps;
  const bool pre = !c.no_pre_norm;      // false: the sublayers read the residual itself, h = T(x)
  auto mwp = [&](int which) { return (const T*)m->mw[which - DN_SQ_EMBED]; };
  auto write_back = [&](const T* mix, const T* out) {
    if (W % 4 == 0) return launch(k_write_back<T, 4>, dim3(ew4), dim3(256), 0, s, m->xs, N, W, S, mix, out, (const float*)m->y);
    return launch(k_write_back<T, 1>, dim3(ew), dim3(256), 0, s, m->xs, N, W, S, mix, out, (const float*)m->y);
  };
  // a sublayer's output a y (+ b y2) joins the residual, through the norm after the sublayer where the model has one
  const NextNorm<T> no_next{nullptr, nullptr, nullptr, nullptr};
  // the norm before the sublayer that follows, when the joining kernel can produce it (plain residual, both norms dynamic tanh)
  const bool can_fuse_next = c.post_norm && dyt && S <= 0;
  auto next_norm = [&](const SeqLayer& nl, int which) {
    return NextNorm<T>{(const T*)nl.w[which], (const T*)nl.w[which == DN_SQ_NORM1 ? DN_SQ_NORM1_B : DN_SQ_NORM2_B],
                       (const T*)nl.w[which == DN_SQ_NORM1 ? DN_SQ_NORM1_ALPHA : DN_SQ_NORM2_ALPHA], (T*)m->h};
  };
  const MoeSrc<T> no_moe{nullptr, nullptr, nullptr, nullptr, 0, 0, nullptr, nullptr, nullptr};
  auto join = [&](SeqLayer& l, int post, int hc_mix, int hc_out, float a, const float* y2, float bb, NextNorm<T> nx, const MoeSrc<T>* ms = nullptr) -> cudaError_t {
    auto w = [&](int i) { return (const T*)l.w[i]; };
    if (c.post_norm && !dyt)      // RMS norm of the sublayer's output, added to the plain residual; h = T(x) for a model without norms before
      return launch(k_rms_join<T>, dim3(N), nthr, nsm, s, m->xs, W, ms ? (const float*)nullptr : (const float*)m->y, a, y2, bb,
                    ms ? *ms : no_moe, w(post), 1, c.eps, pre ? (T*)nullptr : (T*)m->h);
    if (c.post_norm) {
      if (S <= 0) return launch(k_dyt_add<T>, dim3(ew), dim3(256), 0, s, m->xs, NW, W, (const float*)m->y, a, y2, bb, w(post), w(post + 1), w(post + 2), nx);
      cudaError_t e = launch(k_dyt_inplace<T>, dim3(ew), dim3(256), 0, s, m->y, NW, W, a, y2, bb, w(post), w(post + 1), w(post + 2));
      if (e != cudaSuccess) return e;
    } else if (y2 || a != 1.f) {
      cudaError_t e = launch(k_axpby, dim3(ew), dim3(256), 0, s, m->y, NW, a, y2 ? y2 : (const float*)m->y, y2 ? bb : 0.f);
      if (e != cudaSuccess) return e;
    }
    return write_back(w(hc_mix), w(hc_out));
  };
#define PH(id) CK(mark(m, id, s))
  PH(DN_SEQ_PH_EMBED);
  CK(launch(k_embed<T>, dim3(N), dim3(128), 0, s, (const T*)m->embed, b, c.embed_scale, W, S1, m->xs, mwp(DN_SQ_EMBED_NORM), mwp(DN_SQ_EMBED_NORM_B),
            c.embed_norm ? mwp(DN_SQ_EMBED_NORM_ALPHA) : (const T*)nullptr, m->x0, pre ? (T*)nullptr : (T*)m->h,
            c.bigram_buckets > 0 ? mwp(DN_SQ_BIGRAM) : (const T*)nullptr));
  // the norm before a sublayer and, where the model has them, the sublayer's input convolution with its carried rows
  auto norm_in = [&](SeqLayer& l, const Run& run, int q) -> int {
    auto w = [&](int i) { return (const T*)l.w[i]; };
    const int nrm = q == 0 ? DN_SQ_NORM1 : DN_SQ_NORM2, nb = q == 0 ? DN_SQ_NORM1_B : DN_SQ_NORM2_B, na = q == 0 ? DN_SQ_NORM1_ALPHA : DN_SQ_NORM2_ALPHA;
    const bool fused = taps > 0 && b.max_len == 1;      // every entry one token: the norm kernel convolves and carries the row itself
    T* dst = taps > 0 && !fused ? (T*)m->hn : (T*)m->h;
    T* cst = taps > 0 ? (T*)m->conv_state + run.canon_off[q] : (T*)nullptr;
    const T* cwq = taps > 0 ? w(q == 0 ? DN_SQ_CANON1 : DN_SQ_CANON2) : (const T*)nullptr;
    CK(launch(k_read_norm<T>, dim3(N), nthr, nsm, s, m->xs, N, W, S, w(q == 0 ? DN_SQ_HC1_IN : DN_SQ_HC2_IN), w(nrm), dyt ? 0 : 1, 0, c.eps, (const int32_t*)nullptr, dst,
              w(nb), dyt ? w(na) : (const T*)nullptr, lnorm, fused ? cwq : (const T*)nullptr, taps, b.slot, cst, m->conv_stride));
    if (taps > 0 && !fused) {
      CK(mark(m, DN_SEQ_PH_CANON, s));
      const int thr = 128, per = thr * (16 / (int)sizeof(T));
      CK(launch(k_canon<T>, dim3((N + CANON_TOK - 1) / CANON_TOK, (W + per - 1) / per), dim3(thr), 0, s, (const T*)m->hn, cwq, taps, b, W, (const T*)cst, m->conv_stride, (T*)m->h));
      if (taps > 1) {
        CarrySrc<T> cs{{(const T*)m->hn, nullptr, nullptr}, {W, 0, 0}};
        CK(launch(k_conv_carry<T>, dim3((W + 127) / 128, b.E, 1), dim3(128), 0, s, cs, taps, b, cst, m->conv_stride));
      }
    }
    return DN_OK;
  };
  bool h_ready = !pre;
  for (int ri = 0; ri < (int)m->runs.size(); ri++) {
    const Run& run = m->runs[ri];
    SeqLayer& l = m->L[run.layer];
    const dn_seq_layer_cfg& lc = l.c;
    auto w = [&](int i) { return (const T*)l.w[i]; };
    auto wm = [&](int i) { return l.tm_ok[i] ? &l.tm[i] : (const CUtensorMap*)nullptr; };
    if (run.inject) {       // a pass of the loop starts: x <- W_in [x; x0]
      PH(DN_SEQ_PH_OTHER);
      CK(launch(k_loop_cat<T>, dim3((unsigned)((2 * NW + 255) / 256)), dim3(256), 0, s, (const float*)m->xs, (const float*)m->x0, N, W, (T*)m->cat));
      CK(linear<T>(m, s, (const T*)m->cat, m->mw[DN_SQ_LOOP_IN - DN_SQ_EMBED], nullptr, m->xs, N, W, 2 * W, true, 0,
                   LinMaps{m->tm_loop_ok ? &m->tm_loop_in : nullptr, nullptr, &m->x_cat}));
    }
    // ---- mixer sublayer
    PH(DN_SEQ_PH_NORM);
    if (!pre) {
      if (!h_ready || run.inject) CK(launch(k_cast<T>, dim3(ew), dim3(256), 0, s, (const float*)m->xs, NW, (T*)m->h));
    } else if (!h_ready || run.inject) {
      const int rc = norm_in(l, run, 0);
      if (rc != DN_OK) return rc;
    }
    h_ready = false;
    // what the join after this run's last sublayer can prepare: the next run's first norm, unless a loop pass starts there
    const bool next_ok = can_fuse_next && ri + 1 < (int)m->runs.size() && !m->runs[ri + 1].inject;
    const NextNorm<T> nx_run = next_ok ? next_norm(m->L[m->runs[ri + 1].layer], DN_SQ_NORM1) : no_next;
    T* cst = (T*)m->conv_state + run.conv_off;
    float* st = m->delta_state + run.state_off;
    const bool few = N <= 8;      // a decode step: all projections of the mixer in one launch of the row kernel
    float ja = 1.f, jb = 0.f;
    const float* jy2 = nullptr;
    LinSegs sg;
    memset(&sg, 0, sizeof(sg));
    auto add = [&](const void* x, int which, void* y, int rows, int o32) {
      if (rows <= 0) return;
      sg.X[sg.n] = x; sg.W[sg.n] = l.w[which]; sg.Y[sg.n] = y; sg.O[sg.n] = rows; sg.out32[sg.n] = o32; sg.act[sg.n] = ACT_NONE; sg.n++;
    };
    auto run_segs = [&]() {
      int blocks = 0;
      for (int i = 0; i < sg.n; i++) blocks += (sg.O[i] + 7) / 8;
      return launch(k_linear_rows_multi<T>, dim3(blocks), dim3(256), 0, s, (const T*)m->h, sg, N, W);
    };
    if (lc.mixer == DN_MIX_ATTENTION || lc.mixer == DN_MIX_DELTA || lc.mixer == DN_MIX_PARALLEL) {
      PH(DN_SEQ_PH_PROJ);
      if (few) {
        add(nullptr, DN_SQ_Q, m->uq, l.Cq, 0); add(nullptr, DN_SQ_K, m->uk, l.Ck, 0); add(nullptr, DN_SQ_V, m->uv, l.Cv, 0);
        if (lc.mixer == DN_MIX_DELTA) { add(nullptr, DN_SQ_A, m->pa, lc.heads, 1); add(nullptr, DN_SQ_B, m->pb, lc.heads, 1); add(nullptr, DN_SQ_G, m->gt, l.Co, 0); }
        if (lc.mixer != DN_MIX_DELTA && lc.out_gate) add(nullptr, DN_SQ_HEAD_GATE, m->pa, lc.heads, 1);
        CK(run_segs());
      } else {
        CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_Q], nullptr, m->uq, N, l.Cq, W, false, 0, LinMaps{wm(DN_SQ_Q), nullptr, &m->x_h}));
        if (l.Ck) CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_K], nullptr, m->uk, N, l.Ck, W, false, 0, LinMaps{wm(DN_SQ_K), nullptr, &m->x_h}));
        if (l.Cv) CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_V], nullptr, m->uv, N, l.Cv, W, false, 0, LinMaps{wm(DN_SQ_V), nullptr, &m->x_h}));
        if (lc.mixer != DN_MIX_DELTA && lc.out_gate)
          CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_HEAD_GATE], nullptr, m->pa, N, lc.heads, W, true, 0, LinMaps{wm(DN_SQ_HEAD_GATE), nullptr, &m->x_h}));
      }
    }
    if (lc.mixer == DN_MIX_ATTENTION || lc.mixer == DN_MIX_PARALLEL) {
      AttnPrep a{lc.heads, lc.kv_heads, lc.dim, lc.vdim, lc.conv, lc.rot_dims, l.Ck ? 1 : 0, lc.qk_norm, c.eps, l.inv_freq,
                 lc.v_is_k ? 0 : 1, lc.rot_layout == DN_ROT_HALF ? 1 : 0, lc.yarn_factor > 0.f ? 0.1f * logf(lc.yarn_factor) + 1.f : 1.f,
                 lc.qtemp_coef, lc.qtemp_every};
      // values that are the keys: the value pool is the key pool (row stride G dk); the pooled rows likewise
      const void* vpl = lc.v_is_k ? m->kpool[run.kv_index] : m->vpool[run.kv_index];
      void* pkp = m->pkpool[run.kv_index];
      void* pvp = lc.v_is_k ? pkp : m->pvpool[run.kv_index];
      const int Ckk = lc.kv_heads * lc.dim;
      AttnExtra ex{lc.softcap, lc.sink ? l.w[DN_SQ_SINK] : nullptr, lc.out_gate ? (const float*)m->pa : nullptr, lc.mask_kind == DN_MASK_WINDOW ? 1 : 0,
                   lc.v_is_k ? Ckk : 0, lc.pool, pkp, pvp};
      const size_t sm = ((size_t)l.Cq + l.Ck + 40 + lc.heads + lc.kv_heads + lc.rot_dims) * 4;
      PH(DN_SEQ_PH_ATTN_PREP);
      CK(launch(k_attn_prep<T>, dim3(N), dim3(256), sm, s, a, b, (const T*)m->uq, (const T*)m->uk, (const T*)m->uv, w(DN_SQ_Q_CONV),
                w(DN_SQ_K_CONV), w(DN_SQ_V_CONV), w(DN_SQ_Q_NORM), w(DN_SQ_K_NORM), (const T*)cst, m->conv_stride, (T*)m->qb,
                (T*)m->kpool[run.kv_index], (T*)m->vpool[run.kv_index]));
      if (lc.pool > 0)      // blocks that this step's tokens complete get their mean key and value
        CK(launch(k_pool_rows<T>, dim3(N), dim3(128), 0, s, b, lc.pool, Ckk, lc.v_is_k ? 0 : lc.kv_heads * lc.vdim, (const T*)m->kpool[run.kv_index], (const T*)vpl,
                  (T*)pkp, (T*)pvp));
      PH(DN_SEQ_PH_ATTN);
      if (attn_tiles_ok<T>(lc, b))
        CK(attn_tiles(s, b, (const bf16*)m->qb, (const bf16*)m->kpool[run.kv_index], (const bf16*)vpl, lc, ex, (bf16*)m->mo));
      else {
        // a small step (decode): long rows are split over up to AT_MAX_SPLITS blocks, joined by k_attn_merge
        const int Z = N <= AT_SPLIT_ROWS ? AT_MAX_SPLITS : 1;
        CK(launch(k_attn<T, 8>, dim3(N, lc.heads, Z), dim3(AT_WARPS * 32), (size_t)(((lc.dim + 3) & ~3) + AT_WARPS * (2 + (lc.vdim + 31) / 32 * 32)) * 4, s, b,
                  (const T*)m->qb, (const T*)m->kpool[run.kv_index],
                  (const T*)vpl, lc.heads, lc.kv_heads, lc.dim, lc.vdim, lc.chunk, lc.scale, ex, (T*)m->mo, m->attn_part));
        if (Z > 1) CK(launch(k_attn_merge<T>, dim3(N, lc.heads), dim3(128), 0, s, b, lc.heads, lc.vdim, lc.chunk, Z, ex, (const float*)m->attn_part, (T*)m->mo));
      }
    } else if (lc.mixer == DN_MIX_LATENT) {
      // projections: q (or its latent, normed, then up), the key/value latent row, the heads' gates
      const int R = lc.kv_rank, dr = lc.rot_part, dq = lc.dim + dr;
      PH(DN_SEQ_PH_PROJ);
      void* q1 = lc.q_rank > 0 ? m->lr : m->uq;
      const int q1w = lc.q_rank > 0 ? lc.q_rank : l.Cq, q1t = lc.q_rank > 0 ? DN_SQ_DQ : DN_SQ_Q;
      if (few) {
        add(nullptr, q1t, q1, q1w, 0); add(nullptr, DN_SQ_DKV, m->uk, l.Ck, 0);
        if (lc.out_gate) add(nullptr, DN_SQ_HEAD_GATE, m->pa, lc.heads, 1);
        CK(run_segs());
      } else {
        CK(linear<T>(m, s, (const T*)m->h, l.w[q1t], nullptr, q1, N, q1w, W, false, 0, LinMaps{wm(q1t), nullptr, &m->x_h}));
        CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_DKV], nullptr, m->uk, N, l.Ck, W, false, 0, LinMaps{wm(DN_SQ_DKV), nullptr, &m->x_h}));
        if (lc.out_gate)
          CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_HEAD_GATE], nullptr, m->pa, N, lc.heads, W, true, 0, LinMaps{wm(DN_SQ_HEAD_GATE), nullptr, &m->x_h}));
      }
      if (lc.q_rank > 0) {
        CK(launch(k_rms_rows<T>, dim3(N), dim3(128), 0, s, (T*)m->lr, lc.q_rank, w(DN_SQ_DQ_NORM), c.eps));
        CK(linear<T>(m, s, (const T*)m->lr, l.w[DN_SQ_Q], nullptr, m->uq, N, l.Cq, lc.q_rank, false, 0, LinMaps{wm(DN_SQ_Q), nullptr, &l.x_lr}));
      }
      PH(DN_SEQ_PH_LATENT_IN);
      LatentPrep a{lc.heads, lc.dim, dr, R, lc.rot_dims, lc.rot_layout == DN_ROT_HALF ? 1 : 0, c.eps, l.inv_freq};
      T* pool = (T*)m->kpool[run.kv_index];
      CK(launch(k_latent_prep<T>, dim3(N), dim3(256), 0, s, a, b, (const T*)m->uq, (const T*)m->uk, w(DN_SQ_DKV_NORM), (T*)m->qb, pool));
      // the unrotated query parts into the latent space: qb[n, h, 0:R] = W_uk,h^T q[n, h, 0:dim]
      // (all strides multiples of 8 numbers: 16-byte operand rows for the MMA form)
      const bool heads_mma = std::is_same<T, bf16>::value && N >= 16 && dq % 8 == 0 && lc.dim % 8 == 0 && R % 8 == 0 && dr % 8 == 0 && lc.vdim % 8 == 0;
      if (few && (size_t)N * lc.dim * 4 <= 40 * 1024)
        CK(launch(k_absorb_few<T>, dim3((R + 31) / 32, lc.heads), dim3(128), (size_t)(N * lc.dim + 4 * 8 * 32) * 4, s, (const T*)m->uq, w(DN_SQ_UK), (T*)m->qb, N, lc.heads,
                  lc.dim, dq, R, l.Ck));
      else if (heads_mma)
        CK(launch(k_heads_mma<true>, dim3((R + 127) / 128, (N + 63) / 64, lc.heads), dim3(128), 0, s, (const bf16*)m->uq, (const bf16*)l.w[DN_SQ_UK], (bf16*)m->qb, N, R,
                  lc.dim, HeadsGeom{l.Cq, dq, l.Cql, l.Ck, (size_t)lc.dim * R, 1, R}));
      else
        CK(launch(k_linear_heads<T>, dim3((R + 63) / 64, (N + 63) / 64, lc.heads), dim3(256), 0, s, (const T*)m->uq, w(DN_SQ_UK), (T*)m->qb, N, R, lc.dim,
                  HeadsGeom{l.Cq, dq, l.Cql, l.Ck, (size_t)lc.dim * R, 1, R}));
      // multi-query attention of all heads over the cached rows: keys [R + dr], values = their first R numbers
      PH(DN_SEQ_PH_ATTN);
      AttnExtra ex{lc.softcap, nullptr, lc.out_gate ? (const float*)m->pa : nullptr, lc.mask_kind == DN_MASK_WINDOW ? 1 : 0, l.Ck};
      if (std::is_same<T, bf16>::value && latent_tiles_ok(b, l.Ck, R) && (b.max_len >= 16 || b.max_len == 1))
        CK(latent_tiles(s, b, (const bf16*)m->qb, (const bf16*)pool, lc.heads, l.Ck, R, lc.chunk, lc.scale, ex, (bf16*)m->gt, m->attn_part, 2 + m->part_dv));
      else {
        const int Z = N <= AT_SPLIT_ROWS ? AT_MAX_SPLITS : 1;
        const size_t sm = (size_t)(((l.Ck + 3) & ~3) + AT_WARPS * (2 + (R + 31) / 32 * 32)) * 4;
        if (R <= 256)
          CK(launch(k_attn<T, 8>, dim3(N, lc.heads, Z), dim3(AT_WARPS * 32), sm, s, b, (const T*)m->qb, (const T*)pool, (const T*)pool, lc.heads, 1, l.Ck, R,
                    lc.chunk, lc.scale, ex, (T*)m->gt, m->attn_part));
        else
          CK(launch(k_attn<T, 16>, dim3(N, lc.heads, Z), dim3(AT_WARPS * 32), sm, s, b, (const T*)m->qb, (const T*)pool, (const T*)pool, lc.heads, 1, l.Ck, R,
                    lc.chunk, lc.scale, ex, (T*)m->gt, m->attn_part));
        if (Z > 1) CK(launch(k_attn_merge<T>, dim3(N, lc.heads), dim3(128), 0, s, b, lc.heads, R, lc.chunk, Z, ex, (const float*)m->attn_part, (T*)m->gt));
      }
      // out of the latent space: mo[n, h, :] = W_uv,h gt[n, h, :]
      PH(DN_SEQ_PH_LATENT_OUT);
      if (few)
        CK(launch(k_upv_few<T>, dim3((l.Co + 7) / 8), dim3(256), 0, s, (const T*)m->gt, w(DN_SQ_UV), (T*)m->mo, N, lc.heads, lc.vdim, R));
      else if (heads_mma)
        CK(launch(k_heads_mma<false>, dim3((lc.vdim + 127) / 128, (N + 63) / 64, lc.heads), dim3(128), 0, s, (const bf16*)m->gt, (const bf16*)l.w[DN_SQ_UV], (bf16*)m->mo, N,
                  lc.vdim, R, HeadsGeom{l.Col, R, l.Co, lc.vdim, (size_t)lc.vdim * R, R, 1}));
      else
        CK(launch(k_linear_heads<T>, dim3((lc.vdim + 63) / 64, (N + 63) / 64, lc.heads), dim3(256), 0, s, (const T*)m->gt, w(DN_SQ_UV), (T*)m->mo, N, lc.vdim, R,
                  HeadsGeom{l.Col, R, l.Co, lc.vdim, (size_t)lc.vdim * R, R, 1}));
    } else if (lc.mixer == DN_MIX_DELTA) {
      if (!few) {
        CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_A], nullptr, m->pa, N, lc.heads, W, true, 0, LinMaps{wm(DN_SQ_A), nullptr, &m->x_h}));
        CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_B], nullptr, m->pb, N, lc.heads, W, true, 0, LinMaps{wm(DN_SQ_B), nullptr, &m->x_h}));
        CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_G], nullptr, m->gt, N, l.Co, W, false, 0, LinMaps{wm(DN_SQ_G), nullptr, &m->x_h}));
      }
      DeltaPrep a{lc.heads, lc.kv_heads, lc.dim, lc.vdim, lc.conv};
      PH(DN_SEQ_PH_DELTA_PREP);
      CK(launch(k_delta_prep<T>, dim3(N), dim3(256), (size_t)2 * l.Cq * 4, s, a, b, (const T*)m->uq, (const T*)m->uk, (const T*)m->uv,
                w(DN_SQ_Q_CONV), w(DN_SQ_K_CONV), w(DN_SQ_V_CONV), (const float*)m->pa, (const float*)m->pb, w(DN_SQ_A_LOG),
                w(DN_SQ_DT_BIAS), (const T*)cst, m->conv_stride, m->qn, m->kn, m->vv, m->beta, m->decay));
      int R, P;
      recur_shape(lc.dim, &R, &P);
      dim3 grid(b.E * lc.heads, (lc.vdim + 31) / 32);
      // tokens per staged tile: two tiles of `per` floats a token within ~36 KB of shared memory
      const int per = 2 * P * (R + 4) + 36, TB = std::max(1, std::min(16, 4500 / per));
      const size_t dsm = (size_t)2 * TB * per * 4;
#define DR(Rv, Pv) if (R == Rv && P == Pv) CK(launch(k_delta_rule<Rv, Pv>, grid, dim3(32 * Pv), dsm, s, b, lc.heads, lc.kv_heads, lc.dim, lc.vdim, TB, \
                         (const float*)m->qn, (const float*)m->kn, (const float*)m->vv, (const float*)m->beta, (const float*)m->decay, st,      \
                         m->delta_stride, m->od))
      PH(DN_SEQ_PH_DELTA_RULE);
      DR(8, 1); DR(8, 2); DR(8, 4); DR(8, 8); DR(16, 8); DR(16, 16); DR(16, 32); DR(32, 32);
#undef DR
      PH(DN_SEQ_PH_DELTA_OUT);
      CK(launch(k_delta_out<T>, dim3(N, lc.heads), dim3(32), 0, s, (const float*)m->od, (const T*)m->gt, w(DN_SQ_OUT_NORM), lc.heads, lc.vdim,
                c.eps, (T*)m->mo, 0, 0));
    } else {     // DN_MIX_WKV: token-shifted inputs, projections of each, the recurrence read with a bonus
      PH(DN_SEQ_PH_PROJ);
      ShiftMu<T> mu{{w(DN_SQ_MU_R), w(DN_SQ_MU_K), w(DN_SQ_MU_V), w(DN_SQ_MU_G), w(DN_SQ_MU_W)}, 5};
      const size_t xs_ = (size_t)m->MB * W;
      T* xm = (T*)m->xm;
      CK(launch(k_shift_mix<T>, dim3(N), dim3(256), 0, s, (const T*)m->h, b, W, mu, (const T*)cst, m->conv_stride, xm, xs_));
      ShiftCarry<T> carry{nullptr, cst, m->conv_stride, W, b.first, b.slot};
      if (few) {      // one launch for all five projections (the decay's inner one with its tanh); the prep kernel carries the row
        add(xm, DN_SQ_Q, m->uq, l.Cq, 0); add(xm + xs_, DN_SQ_K, m->uk, l.Ck, 0); add(xm + 2 * xs_, DN_SQ_V, m->uv, l.Cv, 0);
        add(xm + 3 * xs_, DN_SQ_G, m->gt, l.Co, 0); add(xm + 4 * xs_, DN_SQ_DECAY1, m->lr, lc.rank, 0);
        sg.act[sg.n - 1] = ACT_TANH;
        CK(run_segs());
        carry.h = (const T*)m->h;
      } else {
        CK(launch(k_shift_carry<T>, dim3((W + 255) / 256, b.E), dim3(256), 0, s, (const T*)m->h, b, W, cst, m->conv_stride));
        CK(linear<T>(m, s, xm, l.w[DN_SQ_Q], nullptr, m->uq, N, l.Cq, W, false, 0, LinMaps{wm(DN_SQ_Q), nullptr, &m->x_xm[0]}));
        CK(linear<T>(m, s, xm + xs_, l.w[DN_SQ_K], nullptr, m->uk, N, l.Ck, W, false, 0, LinMaps{wm(DN_SQ_K), nullptr, &m->x_xm[1]}));
        CK(linear<T>(m, s, xm + 2 * xs_, l.w[DN_SQ_V], nullptr, m->uv, N, l.Cv, W, false, 0, LinMaps{wm(DN_SQ_V), nullptr, &m->x_xm[2]}));
        CK(linear<T>(m, s, xm + 3 * xs_, l.w[DN_SQ_G], nullptr, m->gt, N, l.Co, W, false, 0, LinMaps{wm(DN_SQ_G), nullptr, &m->x_xm[3]}));
      }
      if (!few) CK(linear<T>(m, s, xm + 4 * xs_, l.w[DN_SQ_DECAY1], nullptr, m->lr, N, lc.rank, W, false, ACT_TANH, LinMaps{wm(DN_SQ_DECAY1), nullptr, &m->x_xm[4]}));
      CK(linear<T>(m, s, (const T*)m->lr, l.w[DN_SQ_DECAY2], nullptr, m->dz, N, l.Cq, lc.rank, true, 0, LinMaps{wm(DN_SQ_DECAY2), nullptr, &l.x_lr}));
      PH(DN_SEQ_PH_RECUR_PREP);
      CK(launch(k_decay_prep<T>, dim3(N), dim3(256), 0, s, RECUR_BONUS, N, l.Cq, l.Cv, (const T*)m->uq, (const T*)m->uk, (const T*)m->uv, w(DN_SQ_DECAY_B),
                1.f, 1.f, m->qn, m->kn, m->vv, m->dz, carry));
      PH(DN_SEQ_PH_RECUR);
      { const int rc = decay_rule(m, b, RECUR_BONUS, lc.heads, lc.dim, lc.vdim, l.w[DN_SQ_BONUS], st, s); if (rc != DN_OK) return rc; }
      PH(DN_SEQ_PH_RECUR_OUT);
      CK(launch(k_delta_out<T>, dim3(N, lc.heads), dim3(32), 0, s, (const float*)m->od, (const T*)m->gt, w(DN_SQ_OUT_NORM), lc.heads, lc.vdim,
                c.eps, (T*)m->mo, lc.vdim, 0));
    }
    if (lc.conv > 1) {
      PH(DN_SEQ_PH_CARRY);
      CarrySrc<T> cs{{(const T*)m->uq, (const T*)m->uk, (const T*)m->uv}, {l.Cq, l.Ck, l.Cv}};
      CK(launch(k_conv_carry<T>, dim3((std::max(l.Cq, std::max(l.Ck, l.Cv)) + 127) / 128, b.E, 3), dim3(128), 0, s, cs, lc.conv, b, cst, m->conv_stride));
    }
    PH(DN_SEQ_PH_OUT_PROJ);
    CK(linear<T>(m, s, (const T*)m->mo, l.w[DN_SQ_O], nullptr, m->y, N, W, l.Co, true, 0, LinMaps{wm(DN_SQ_O), nullptr, &l.x_mo}));
    if (lc.mixer == DN_MIX_PARALLEL && lc.r_kind == DN_RIGHT_GDELTA) {     // the generalized delta rule, on the same input
      PH(DN_SEQ_PH_PROJ);
      if (few) {
        memset(&sg, 0, sizeof(sg));
        add(nullptr, DN_SQ_R_Q, m->uq, l.Rc, 0); add(nullptr, DN_SQ_R_K, m->uk, l.Rc, 0); add(nullptr, DN_SQ_R_V, m->uv, l.Rv, 0);
        add(nullptr, DN_SQ_R_G, m->gt, l.Rv, 0); add(nullptr, DN_SQ_R_A, m->aun, l.Rc, 1); add(nullptr, DN_SQ_DECAY1, m->lr, lc.rank, 0);
        sg.act[sg.n - 1] = ACT_TANH;
        CK(run_segs());
      } else {
        CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_R_Q], nullptr, m->uq, N, l.Rc, W, false, 0, LinMaps{wm(DN_SQ_R_Q), nullptr, &m->x_h}));
        CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_R_K], nullptr, m->uk, N, l.Rc, W, false, 0, LinMaps{wm(DN_SQ_R_K), nullptr, &m->x_h}));
        CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_R_V], nullptr, m->uv, N, l.Rv, W, false, 0, LinMaps{wm(DN_SQ_R_V), nullptr, &m->x_h}));
        CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_R_G], nullptr, m->gt, N, l.Rv, W, false, 0, LinMaps{wm(DN_SQ_R_G), nullptr, &m->x_h}));
        CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_R_A], nullptr, m->aun, N, l.Rc, W, true, 0, LinMaps{wm(DN_SQ_R_A), nullptr, &m->x_h}));
        CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_DECAY1], nullptr, m->lr, N, lc.rank, W, false, ACT_TANH, LinMaps{wm(DN_SQ_DECAY1), nullptr, &m->x_h}));
      }
      CK(linear<T>(m, s, (const T*)m->lr, l.w[DN_SQ_DECAY2], nullptr, m->dz, N, l.Rc, lc.rank, true, 0, LinMaps{wm(DN_SQ_DECAY2), nullptr, &l.x_lr}));
      PH(DN_SEQ_PH_RECUR_PREP);
      // few tokens: the heads spread over blocks of four warps; many: one block of up to eight warps a token
      const int gw = std::min(N <= 64 ? 4 : 8, lc.r_heads);
      CK(launch(k_gdelta_prep<T>, dim3(N, N <= 64 ? (lc.r_heads + gw - 1) / gw : 1), dim3(32 * gw), 0, s, lc.r_heads, lc.r_dim, (const T*)m->uq, (const T*)m->uk, (const T*)m->uv,
                w(DN_SQ_DECAY_B), w(DN_SQ_R_AB), m->qn, m->kn, m->vv, m->dz, m->un, m->aun));
      PH(DN_SEQ_PH_RECUR);
      {
        // rows a lane (R), lanes a column (P), columns a block.  The token loop is bound by the latency of its dependent
        // instructions, so a model with few heads (fewer blocks of 16 columns than the GPU has SMs) takes 4 rows a lane and 8
        // columns a block: four times the warps.  A function of the model's sizes only: the order of the sums does not
        // depend on the batch.
        static const int RPC[9][4] = {{4, 4, 1, 32}, {8, 4, 2, 16}, {16, 4, 4, 8}, {32, 4, 8, 8}, {64, 4, 16, 8}, {128, 8, 16, 8}, {256, 8, 32, 8},
                                      {512, 16, 32, 8}, {1024, 32, 32, 8}};
        int R = 32, P = 32, cols = 8;
        if (lc.r_heads * ((lc.r_dim + 15) / 16) < 148) {
          for (int i = 8; i >= 0; i--) if (lc.r_dim <= RPC[i][0]) { R = RPC[i][1]; P = RPC[i][2]; cols = RPC[i][3]; }
        } else {
          recur_shape(lc.r_dim, &R, &P);
          cols = P >= 2 ? 16 : 32;
        }
        const int dv = lc.r_dim;
        dim3 grid(b.E * lc.r_heads, (dv + cols - 1) / cols);
        const int per = 5 * P * (R == 4 ? 4 : R + 4) + cols;
        const int TB = std::max(1, std::min(16, 5800 / per));      // two tiles within ~46 KB of shared memory
        const size_t dsm = (size_t)2 * TB * per * 4;
#define GD(Rv_, Pv_, Cv_) if (R == Rv_ && P == Pv_) CK(launch(k_gdelta_rule<Rv_, Pv_, Cv_>, grid, dim3(Cv_ * Pv_), dsm, s, b, lc.r_heads, lc.r_dim, dv, TB, \
                           (const float*)m->qn, (const float*)m->kn, (const float*)m->vv, (const float*)m->dz, (const float*)m->un, (const float*)m->aun, st, \
                           m->delta_stride, m->od))
#define GD2(Rv_, Pv_, Cv_) if (cols == Cv_) GD(Rv_, Pv_, Cv_)
        GD(4, 1, 32); GD(4, 2, 16); GD(4, 4, 8); GD(4, 8, 8); GD(4, 16, 8); GD(8, 16, 8); GD(8, 32, 8); GD2(16, 32, 8); GD2(32, 32, 8);
        GD(8, 1, 32); GD(8, 2, 16); GD(8, 4, 16); GD(8, 8, 16); GD(16, 8, 16); GD(16, 16, 16); GD2(16, 32, 16); GD2(32, 32, 16);
#undef GD2
#undef GD
      }
      PH(DN_SEQ_PH_RECUR_OUT);
      CK(launch(k_delta_out<T>, dim3(N, lc.r_heads), dim3(32), 0, s, (const float*)m->od, (const T*)m->gt, w(DN_SQ_R_NORM), lc.r_heads, lc.r_dim,
                c.eps, (T*)m->mo, lc.r_dim, 1));
      PH(DN_SEQ_PH_OUT_PROJ);
      CK(linear<T>(m, s, (const T*)m->mo, l.w[DN_SQ_R_O], nullptr, m->y2, N, W, l.Rv, true, 0, LinMaps{wm(DN_SQ_R_O), nullptr, &l.x_mo_r}));
      ja = lc.left_scale; jb = lc.right_scale; jy2 = m->y2;
    } else if (lc.mixer == DN_MIX_PARALLEL) {     // the linear-attention half, on the same input; its scratch is free again
      PH(DN_SEQ_PH_PROJ);
      if (few) {
        memset(&sg, 0, sizeof(sg));
        add(nullptr, DN_SQ_R_Q, m->uq, l.Rc, 0); add(nullptr, DN_SQ_R_K, m->uk, l.Rc, 0); add(nullptr, DN_SQ_R_V, m->uv, l.Rv, 0);
        add(nullptr, DN_SQ_R_G, m->gt, l.Rv, 0); add(nullptr, DN_SQ_DECAY1, m->lr, lc.rank, 0);
        CK(run_segs());
      } else {
        CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_R_Q], nullptr, m->uq, N, l.Rc, W, false, 0, LinMaps{wm(DN_SQ_R_Q), nullptr, &m->x_h}));
        CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_R_K], nullptr, m->uk, N, l.Rc, W, false, 0, LinMaps{wm(DN_SQ_R_K), nullptr, &m->x_h}));
        CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_R_V], nullptr, m->uv, N, l.Rv, W, false, 0, LinMaps{wm(DN_SQ_R_V), nullptr, &m->x_h}));
        CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_R_G], nullptr, m->gt, N, l.Rv, W, false, 0, LinMaps{wm(DN_SQ_R_G), nullptr, &m->x_h}));
        CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_DECAY1], nullptr, m->lr, N, lc.rank, W, false, 0, LinMaps{wm(DN_SQ_DECAY1), nullptr, &m->x_h}));
      }
      CK(linear<T>(m, s, (const T*)m->lr, l.w[DN_SQ_DECAY2], nullptr, m->dz, N, l.Rc, lc.rank, true, 0, LinMaps{wm(DN_SQ_DECAY2), nullptr, &l.x_lr}));
      PH(DN_SEQ_PH_RECUR_PREP);
      CK(launch(k_decay_prep<T>, dim3(N), dim3(256), 0, s, RECUR_AFTER, N, l.Rc, l.Rv, (const T*)m->uq, (const T*)m->uk, (const T*)m->uv, w(DN_SQ_DECAY_B),
                1.f / sqrtf((float)lc.r_dim), lc.tau, m->qn, m->kn, m->vv, m->dz, ShiftCarry<T>{nullptr, nullptr, 0, 0, nullptr, nullptr}));
      PH(DN_SEQ_PH_RECUR);
      { const int rc = decay_rule(m, b, RECUR_AFTER, lc.r_heads, lc.r_dim, lc.r_vdim, nullptr, st, s); if (rc != DN_OK) return rc; }
      PH(DN_SEQ_PH_RECUR_OUT);
      CK(launch(k_delta_out<T>, dim3(N, lc.r_heads), dim3(32), 0, s, (const float*)m->od, (const T*)m->gt, w(DN_SQ_R_NORM), lc.r_heads, lc.r_vdim,
                c.eps, (T*)m->mo, 0, 0));
      PH(DN_SEQ_PH_OUT_PROJ);
      CK(linear<T>(m, s, (const T*)m->mo, l.w[DN_SQ_R_O], nullptr, m->y2, N, W, l.Rv, true, 0, LinMaps{wm(DN_SQ_R_O), nullptr, &l.x_mo_r}));
      ja = lc.left_scale; jb = lc.right_scale; jy2 = m->y2;
    }
    PH(DN_SEQ_PH_WRITE_BACK);
    const NextNorm<T> nx_mix = lc.ff > 0 ? (can_fuse_next ? next_norm(l, DN_SQ_NORM2) : no_next) : nx_run;
    if (lc.mixer == DN_MIX_PARALLEL && lc.branch_norm)
      CK(launch(k_rms2_join<T>, dim3(N), nthr, 0, s, m->xs, W, (const float*)m->y, ja, w(DN_SQ_L_OUT), jy2, jb, w(DN_SQ_R_OUT), c.eps));
    else
      CK(join(l, DN_SQ_POST1, DN_SQ_HC1_MIX, DN_SQ_HC1_OUT, ja, jy2, jb, nx_mix));
    if (lc.ff == 0) h_ready = nx_run.alpha != nullptr || !pre;
    // ---- feed-forward sublayer
    if (lc.ff > 0) {
      PH(DN_SEQ_PH_NORM);
      if (!can_fuse_next && pre) {
        const int rc = norm_in(l, run, 1);
        if (rc != DN_OK) return rc;
      }
      if (lc.mlp_kind == DN_MLP_MOE) {
        const bool fused = c.post_norm && S <= 0;
        const bool rmsj = fused && !dyt;      // the RMS join adds the pairs, the identity experts' input and the gated shared expert itself
        const int rc = moe_ff<T>(m, l, N, fused, fused ? nx_run : no_next, s, !rmsj);
        if (rc != DN_OK) return rc;
        if (rmsj) {
          const bool scored = lc.router_kind == DN_ROUTER_SCORED;
          const MoeSrc<T> ms{m->eo, m->rwt, m->rpos, m->ridx, lc.top, scored ? lc.experts : INT32_MAX, (const T*)m->h,
                             lc.shared_ff > 0 ? (const float*)m->y2 : (const float*)nullptr, lc.shared_gate ? (const float*)m->sgate : (const float*)nullptr};
          CK(join(l, DN_SQ_POST2, DN_SQ_HC2_MIX, DN_SQ_HC2_OUT, 1.f, nullptr, 0.f, no_next, &ms));
        } else if (!fused) CK(join(l, DN_SQ_POST2, DN_SQ_HC2_MIX, DN_SQ_HC2_OUT, 1.f, lc.shared_ff > 0 ? (const float*)m->y2 : nullptr, 1.f, nx_run));
        h_ready = nx_run.alpha != nullptr || !pre;
      } else {
        PH(DN_SEQ_PH_FF_UP);
        if (lc.ff_act == DN_FF_RELU2)      // no gate: relu(W_up h + b)^2
          CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_UP], nullptr, m->act, N, lc.ff, W, false, ACT_RELU2, LinMaps{wm(DN_SQ_UP), nullptr, &m->x_h}, 0.f, l.w[DN_SQ_UP_B]));
        else
          CK(linear<T>(m, s, (const T*)m->h, l.w[DN_SQ_GATE], l.w[DN_SQ_UP], m->act, N, lc.ff, W, false, ACT_GEGLU, LinMaps{wm(DN_SQ_GATE), wm(DN_SQ_UP), &m->x_h}));
        PH(DN_SEQ_PH_FF_DOWN);
        CK(linear<T>(m, s, (const T*)m->act, l.w[DN_SQ_DOWN], nullptr, m->y, N, W, lc.ff, true, 0, LinMaps{wm(DN_SQ_DOWN), nullptr, &l.x_act}, 0.f,
                     lc.ff_act == DN_FF_RELU2 ? l.w[DN_SQ_DOWN_B] : nullptr));
        PH(DN_SEQ_PH_WRITE_BACK);
        CK(join(l, DN_SQ_POST2, DN_SQ_HC2_MIX, DN_SQ_HC2_OUT, 1.f, nullptr, 0.f, nx_run));
        h_ready = (nx_run.alpha != nullptr && c.post_norm && S <= 0) || !pre;
      }
    }
    PH(DN_SEQ_PH_OTHER);
    if (trace) CK(launch(k_stream_sum, dim3(ew), dim3(256), 0, s, (const float*)m->xs, N, W, S1, trace + (size_t)ri * N * W));
  }
  if (n_want > 0) {
    PH(DN_SEQ_PH_NORM);
    CK(launch(k_read_norm<T>, dim3(n_want), nthr, nsm, s, m->xs, N, W, S, (const T*)nullptr, (const T*)m->final_norm, dyt ? 0 : 1, 1, c.eps, want_dev, (T*)m->h,
              mwp(DN_SQ_FINAL_NORM_B), dyt ? mwp(DN_SQ_FINAL_NORM_ALPHA) : (const T*)nullptr, lnorm, (const T*)nullptr, 0, (const int32_t*)nullptr, (T*)nullptr,
              (size_t)0));
    PH(DN_SEQ_PH_HEAD);
    CK(linear<T>(m, s, (const T*)m->h, m->head, nullptr, logits, n_want, c.vocab, W, true, 0, LinMaps{m->tm_head_ok ? &m->tm_head : nullptr, nullptr, &m->x_h}));
    if (c.logit_softcap > 0.f)
      CK(launch(k_softcap, dim3((unsigned)(((size_t)n_want * c.vocab + 255) / 256)), dim3(256), 0, s, logits, (size_t)n_want * c.vocab, c.logit_softcap));
    if (c.logit_scale != 0.f && c.logit_scale != 1.f)
      CK(launch(k_scale, dim3((unsigned)(((size_t)n_want * c.vocab + 255) / 256)), dim3(256), 0, s, logits, (size_t)n_want * c.vocab, c.logit_scale));
  }
  PH(DN_SEQ_PH_OTHER);
#undef PH
  return DN_OK;
}

extern "C" int dn_seq_step(dn_seq_model* m, int E, const int32_t* slots, const int32_t* counts, const int32_t* tokens, int n_want,
                           const int32_t* want, float* logits, float* trace, dn_seq_stream sp) {
  if (!m || E <= 0 || !slots || !counts || !tokens || (n_want > 0 && (!want || !logits))) return fail(DN_EINVAL, "bad argument");
  if (E > m->cfg.max_seqs) return fail(DN_EINVAL, "%d entries > %d state slots", E, m->cfg.max_seqs);
  cudaStream_t s = (cudaStream_t)sp;
  int N = 0;
  size_t need = 0;
  for (int e = 0; e < E; e++) {
    const int sl = slots[e];
    if (sl < 0 || sl >= m->cfg.max_seqs || m->length[sl] < 0) return fail(DN_EINVAL, "entry %d: slot %d is not open", e, sl);
    for (int f = 0; f < e; f++) if (slots[f] == sl) return fail(DN_EINVAL, "slot %d appears twice in one step", sl);
    if (counts[e] <= 0) return fail(DN_EINVAL, "entry %d brings no tokens", e);
    N += counts[e];
    const size_t pages = ((size_t)m->length[sl] + counts[e] + PAGE - 1) / PAGE;
    if (pages > (size_t)m->max_pages) return fail(DN_ENOSPC, "sequence too long for the block table");
    if (pages > m->pages[sl].size()) need += pages - m->pages[sl].size();
  }
  if (N > m->MB) return fail(DN_EINVAL, "%d tokens > max_batch_tokens %d", N, m->MB);
  if (n_want > N) return fail(DN_EINVAL, "more wanted rows than tokens");
  for (int i = 0; i < N; i++) if (tokens[i] < 0 || tokens[i] >= m->cfg.vocab) return fail(DN_EINVAL, "token id %d out of range", tokens[i]);
  if (need > m->free_pages.size()) return fail(DN_ENOSPC, "cache pool exhausted: %zu pages needed, %zu free", need, m->free_pages.size());
  for (int i = 0; i < n_want; i++) if (want[i] < 0 || want[i] >= N) return fail(DN_EINVAL, "wanted row %d out of range", want[i]);
  if (!m->embed || !m->final_norm || !m->head) return fail(DN_ENOENT, "embedding / final norm / head are not bound");
  const bool dyt = m->cfg.norm_kind == DN_NORM_DYT;
  auto mhas = [&](int k) { return m->mw[k - DN_SQ_EMBED] != nullptr; };
  if (dyt && (!mhas(DN_SQ_FINAL_NORM_B) || !mhas(DN_SQ_FINAL_NORM_ALPHA))) return fail(DN_ENOENT, "bias / alpha of the final norm are not bound");
  if (m->cfg.embed_norm && (!mhas(DN_SQ_EMBED_NORM) || !mhas(DN_SQ_EMBED_NORM_B) || !mhas(DN_SQ_EMBED_NORM_ALPHA))) return fail(DN_ENOENT, "the embedding's norm is not bound");
  if (m->cfg.loop_times > 0 && !mhas(DN_SQ_LOOP_IN)) return fail(DN_ENOENT, "the loop's input matrix is not bound");
  if (m->cfg.norm_kind == DN_NORM_LAYER && !mhas(DN_SQ_FINAL_NORM_B)) return fail(DN_ENOENT, "the final norm's bias is not bound");
  if (m->cfg.bigram_buckets > 0 && !mhas(DN_SQ_BIGRAM)) return fail(DN_ENOENT, "the bigram table is not bound");
  for (int i = 0; i < m->cfg.n_layers; i++) {
    const SeqLayer& l = m->L[i];
    auto has = [&](int k) { return l.w[k] != nullptr; };
    const int mx = l.c.mixer;
    const bool moe = l.c.mlp_kind == DN_MLP_MOE;
    bool ok = has(DN_SQ_Q) && has(DN_SQ_O);
    if (!m->cfg.no_pre_norm) ok = ok && has(DN_SQ_NORM1) && (l.c.ff == 0 || has(DN_SQ_NORM2));
    if (l.c.ff > 0 && !moe) ok = ok && (l.c.ff_act == DN_FF_RELU2 || has(DN_SQ_GATE)) && has(DN_SQ_UP) && has(DN_SQ_DOWN);
    if (l.c.ff > 0 && moe) {
      ok = ok && has(DN_SQ_ROUTER) && (l.c.shared_ff == 0 || (has(DN_SQ_SH_GATE) && has(DN_SQ_SH_UP) && has(DN_SQ_SH_DOWN)));
      if (l.c.shared_gate) ok = ok && has(DN_SQ_SH_SG);
      for (const void* p : l.etab_h) ok = ok && p != nullptr;
    }
    if (dyt) ok = ok && has(DN_SQ_NORM1_B) && has(DN_SQ_NORM1_ALPHA) && (l.c.ff == 0 || (has(DN_SQ_NORM2_B) && has(DN_SQ_NORM2_ALPHA)));
    if (m->cfg.post_norm) ok = ok && has(DN_SQ_POST1) && (l.c.ff == 0 || has(DN_SQ_POST2));
    if (m->cfg.post_norm && dyt) ok = ok && has(DN_SQ_POST1_B) && has(DN_SQ_POST1_ALPHA) && (l.c.ff == 0 || (has(DN_SQ_POST2_B) && has(DN_SQ_POST2_ALPHA)));
    if (mx == DN_MIX_LATENT) ok = ok && has(DN_SQ_DKV) && has(DN_SQ_DKV_NORM) && has(DN_SQ_UK) && has(DN_SQ_UV) && (!l.c.out_gate || has(DN_SQ_HEAD_GATE)) &&
                                  (l.c.q_rank == 0 || (has(DN_SQ_DQ) && has(DN_SQ_DQ_NORM)));
    else if (l.Ck) ok = ok && has(DN_SQ_K) && (l.c.v_is_k || has(DN_SQ_V));
    if (m->cfg.norm_kind == DN_NORM_LAYER) ok = ok && has(DN_SQ_NORM1_B) && (l.c.ff == 0 || has(DN_SQ_NORM2_B));
    if (m->cfg.canon_taps > 0) ok = ok && has(DN_SQ_CANON1) && (l.c.ff == 0 || has(DN_SQ_CANON2));
    if (l.c.conv > 0) ok = ok && has(DN_SQ_Q_CONV) && (!l.Ck || (has(DN_SQ_K_CONV) && has(DN_SQ_V_CONV)));
    if (mx == DN_MIX_ATTENTION || mx == DN_MIX_PARALLEL) {
      if (l.c.qk_norm) ok = ok && has(DN_SQ_Q_NORM) && (!l.Ck || has(DN_SQ_K_NORM));
      if (l.c.sink) ok = ok && has(DN_SQ_SINK);
      if (l.c.out_gate) ok = ok && has(DN_SQ_HEAD_GATE);
    }
    if (mx == DN_MIX_DELTA) ok = ok && has(DN_SQ_A) && has(DN_SQ_B) && has(DN_SQ_G) && has(DN_SQ_A_LOG) && has(DN_SQ_DT_BIAS) && has(DN_SQ_OUT_NORM);
    if (mx == DN_MIX_PARALLEL) ok = ok && has(DN_SQ_R_Q) && has(DN_SQ_R_K) && has(DN_SQ_R_V) && has(DN_SQ_R_G) && has(DN_SQ_R_O) && has(DN_SQ_R_NORM) &&
                                    has(DN_SQ_DECAY1) && has(DN_SQ_DECAY2) && has(DN_SQ_DECAY_B);
    if (mx == DN_MIX_PARALLEL && l.c.r_kind == DN_RIGHT_GDELTA) ok = ok && has(DN_SQ_R_A) && has(DN_SQ_R_AB);
    if (mx == DN_MIX_PARALLEL && l.c.branch_norm) ok = ok && has(DN_SQ_L_OUT) && has(DN_SQ_R_OUT);
    if (mx == DN_MIX_WKV) ok = ok && has(DN_SQ_G) && has(DN_SQ_OUT_NORM) && has(DN_SQ_DECAY1) && has(DN_SQ_DECAY2) && has(DN_SQ_DECAY_B) && has(DN_SQ_BONUS) &&
                               has(DN_SQ_MU_R) && has(DN_SQ_MU_K) && has(DN_SQ_MU_V) && has(DN_SQ_MU_G) && has(DN_SQ_MU_W);
    if (m->cfg.streams > 0) ok = ok && has(DN_SQ_HC1_IN) && has(DN_SQ_HC1_OUT) && has(DN_SQ_HC1_MIX) &&
                                 (l.c.ff == 0 || (has(DN_SQ_HC2_IN) && has(DN_SQ_HC2_OUT) && has(DN_SQ_HC2_MIX)));
    if (!ok) return fail(DN_ENOENT, "layer %d: not every tensor of the layer is bound", i);
  }
  // the previous step's staging copies must have read the pinned buffers before they are rewritten
  CK(cudaEventSynchronize(m->staged));
  int32_t* h = m->stage_h;
  int32_t *tok = h, *slot = h + N, *pos = h + 2 * N, *first = h + 3 * N, *brow = h + 4 * N, *es = h + 5 * N, *esl = es + E + 1, *ep0 = esl + E, *wr = ep0 + E;
  const dn_seq_cfg& mc = m->cfg;
  int n = 0;
  for (int e = 0; e < E; e++) {
    const int sl = slots[e];
    const size_t pages = ((size_t)m->length[sl] + counts[e] + PAGE - 1) / PAGE;
    const size_t had = m->pages[sl].size();
    while (m->pages[sl].size() < pages) {
      const int pg = m->free_pages.back();
      m->free_pages.pop_back();
      m->bt_h[(size_t)sl * m->max_pages + m->pages[sl].size()] = pg;
      m->pages[sl].push_back(pg);
    }
    if (pages > had)
      CK(cudaMemcpyAsync(m->bt_d + (size_t)sl * m->max_pages + had, m->bt_h + (size_t)sl * m->max_pages + had, (pages - had) * 4,
                         cudaMemcpyHostToDevice, s));
    es[e] = n; esl[e] = sl; ep0[e] = m->length[sl];
    for (int i = 0; i < counts[e]; i++, n++) {
      tok[n] = tokens[n]; slot[n] = sl; pos[n] = m->length[sl] + i; first[n] = es[e];
      // the bigram row: a hash of (previous token, token); the table's last row for a sequence's first token
      const int prev = m->last_tok[sl];
      brow[n] = mc.bigram_buckets <= 0 ? 0 : prev < 0 ? mc.bigram_buckets
              : (int32_t)(((int64_t)prev * mc.bigram_mul_prev + (int64_t)tokens[n] * mc.bigram_mul_cur) % mc.bigram_buckets);
      m->last_tok[sl] = tokens[n];
    }
    m->length[sl] += counts[e];
  }
  es[E] = N;
  for (int i = 0; i < n_want; i++) wr[i] = want[i];
  const size_t ints = 5 * (size_t)N + 3 * (size_t)E + 1 + n_want;
  CK(cudaMemcpyAsync(m->stage_d, h, ints * 4, cudaMemcpyHostToDevice, s));
  CK(cudaEventRecord(m->staged, s));
  int32_t* d = m->stage_d;
  int max_len = 0, row_tiles = 0;
  for (int e = 0; e < E; e++) { max_len = counts[e] > max_len ? counts[e] : max_len; row_tiles += (counts[e] + AT_ROWS - 1) / AT_ROWS; }
  Batch b{d, d + N, d + 2 * N, d + 3 * N, d + 5 * N, d + 5 * N + E + 1, d + 5 * N + 2 * E + 1, m->bt_d, N, E, m->max_pages, max_len, row_tiles, d + 4 * N};
  const int32_t* want_dev = d + 5 * N + 3 * E + 1;
  auto run = [&](float* lg) {
    if (m->cfg.dtype == DN_SEQ_F32) return step_T<float>(m, b, n_want, want_dev, lg, trace, s);
    return step_T<bf16>(m, b, n_want, want_dev, lg, trace, s);
  };
  // (the legacy default stream cannot be captured: steps queued on it are launched one by one)
  const bool capturable = s != nullptr && s != cudaStreamLegacy && s != cudaStreamPerThread;
  if (!(m->graphs_on && capturable && N == E && N <= 8 && !trace && !m->prof_on)) return run(logits);
  // a decode step: replay (capturing at first use) the step's kernels as one graph
  const auto key = std::make_pair(E, n_want);
  auto it = m->graphs.find(key);
  if (it == m->graphs.end()) {
    const long long l0 = g_launches.load();
    if (cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
      cudaGetLastError();          // this stream cannot be captured now (e.g. it is part of the caller's own capture): launch one by one
      return run(logits);
    }
    const int rc = run(m->lg_buf);
    cudaGraph_t graph = nullptr;
    const cudaError_t ec = cudaStreamEndCapture(s, &graph);
    if (rc != DN_OK) { if (graph) cudaGraphDestroy(graph); return rc; }
    if (ec != cudaSuccess) return fail(DN_ECUDA, "graph capture of a decode step failed: %s", cudaGetErrorString(ec));
    cudaGraphExec_t exec = nullptr;
    const cudaError_t ei = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (ei != cudaSuccess) return fail(DN_ECUDA, "graph instantiation failed: %s", cudaGetErrorString(ei));
    const long long per = g_launches.load() - l0;
    g_launches -= per;          // captured, not run: replays are what is counted
    it = m->graphs.emplace(key, std::make_pair(exec, per)).first;
  }
  CK(cudaGraphLaunch(it->second.first, s));
  g_launches += it->second.second;
  if (n_want > 0) CK(cudaMemcpyAsync(logits, m->lg_buf, (size_t)n_want * m->cfg.vocab * 4, cudaMemcpyDeviceToDevice, s));
  return DN_OK;
}

extern "C" int dn_seq_set_graphs(dn_seq_model* m, int on) {
  if (!m) return fail(DN_EINVAL, "null model");
  m->graphs_on = on != 0;
  return DN_OK;
}

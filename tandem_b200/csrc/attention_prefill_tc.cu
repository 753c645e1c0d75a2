// Paged causal attention for prompt portions on the fifth-generation tensor cores (tcgen05), head
// size TB_HD (64 or 128) fixed at compile time.
//
// Work comes in items: up to 2 x (128 / G) consecutive tokens of one request for one kv head (G =
// query heads per kv head), i.e. two query tiles of 128 rows = (token, query head of the group)
// pairs that share the request's keys and values.  One persistent block per SM walks a queue of
// items that the host has balanced (heaviest first, each to the block with the least work so far);
// nothing is fetched or counted at run time, every warp reads the same queue.
//
//   warps 0-3 / 4-7  softmax of tile 0 / tile 1: one query row per thread (a row of the MMA is a
//            lane of tensor memory, a warp reaches the 32 lanes of its number modulo 4).  A thread
//            reads its row of S (128 keys) with tcgen05.ld, masks it at the causal or the window's
//            edge, keeps the running maximum and sum in float32 (exp2), writes the probabilities
//            as bfloat16 pairs over the first half of S (tcgen05.st: the A operand of the second
//            product) and rescales O in tensor memory when the row's reference maximum has to
//            move (only when it grew by more than 2^8 since the reference was set: the sum is
//            kept against the same reference, so the result is exact).  At the item's end it
//            reads O, divides by the sum and writes the output rows.
//   warp 8   brings the item's two query tiles (one 3-D tensor copy per 64 columns: tokens x
//            heads of the group x 64 elements, in the 128-byte-swizzled layout the MMA reads) and
//            streams the keys: stages of 128 keys, a bulk copy per page piece, as the cache's own
//            tile layout (cache_layout.cuh) already is what tcgen05 reads: K a K-major B operand,
//            V an MN-major one;
//   warp 9   streams the values the same way (keys are used early in a step and values late:
//            with rings and barriers of their own neither waits for the other's buffer);
//   warps 10 / 11  one thread each issues the MMAs of tile 0 / tile 1: S = Q K^T (M = 128 rows,
//            N = 128 keys, both operands in shared memory), and when the tile's softmax has
//            handed over the probabilities, O += P V (A from tensor memory) and at once the
//            scores of the next step, sixteen MMAs in a row (a batch of MMAs that finds the
//            tensor cores idle pays some 300 cycles before its first result).  S and P share their
//            columns: the next S overwrites the probabilities that the product issued just before
//            it reads, and MMAs of one thread are executed in the order of issue.  A tile's chain
//            S -> softmax -> P V, S is serial; the two tiles run half a step apart (their warps
//            take turns at the exponentials) and keep the tensor cores and the special-function
//            unit busy in turn.  Tensor memory: S0, S1, O0, O1, 128 columns each.
//
// It stands where 12vivi/tandem calls FlashInfer's paged prefill wrapper
// (python/tandem/layers/flashinfer_attention.py:167-171,194-209); the arithmetic is
// python/tandem/layers/attention.py:46-56 of the reference.
#include <cuda.h>

#include "attention_common.cuh"

namespace tb {

static_assert(HD == 64 || HD == 128, "the tcgen05 prefill kernel takes head sizes 64 and 128");
constexpr int BM = 128;             // rows of a query tile
constexpr int STEP_KEYS = 128;      // keys per stage and per S
#ifndef TB_PF_STAGES
#define TB_PF_STAGES (TB_HD == 128 ? 2 : 4)
#endif
constexpr int KV_STAGES = TB_PF_STAGES;  // of keys, and as many of values
constexpr int SOFTMAX_WARPS = 8, K_WARP = 8, V_WARP = 9, ISSUE_WARP = 10;
constexpr int THREADS = 384;
constexpr int WORK_INTS = 5;        // first token row, request, first position, number of tokens, kv head
constexpr int STAGE_ELEMS_1 = STEP_KEYS * HD, STAGE_BYTES_1 = STAGE_ELEMS_1 * 2;  // K or V of one step
constexpr int Q_BYTES = BM * HD * 2;
constexpr int TMEM_COLS = 512, TMEM_S = 0, TMEM_O = 256, TMEM_TILE = 128;  // S_t at t * 128, O_t at 256 + t * 128
constexpr float RESCALE_AT = 8.f;   // move a row's reference maximum when it has grown by 2^8
constexpr int REGS_SOFTMAX = 224, REGS_OTHER = 56;  // the softmax warps hold a row of 128 scores in registers

struct PrefillArgs {
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  const int* block_table;
  int table_stride;
  const int* work;  // [queue_len][blocks][WORK_INTS]; an item of no tokens ends a block's queue
  int queue_len;
  __nv_bfloat16* out;
  int* status;
  int nh, nkv, page_size, window;
  float scale_log2;
};

// With -DTB_PF_TRACE the first block records when its warps pass the stations of their first 64 steps
// (clock64; tb_attention_prefill_tc_trace reads the record): the timeline the design was read off.
#ifdef TB_PF_TRACE
__device__ long long tb_trace[6 * 64 * 8];
#define TRACE(role, n, ev) do { if (blockIdx.x == 0 && (n) < 64) tb_trace[((role) * 64 + (n)) * 8 + (ev)] = clock64(); } while (0)
#else
#define TRACE(role, n, ev) do { } while (0)
#endif

// What an item means for every warp of the block.
struct Item {
  int t0, req, p0, ntok, kvh;
  int kb, ke, s0, steps;   // keys [kb, ke), steps of 128 keys from s0 on
  int jb0, je0, jb1, je1;  // the steps [jb, je) in which tile 0 / tile 1 has keys of its own
  __device__ __forceinline__ int jb(int t) const { return t ? jb1 : jb0; }
  __device__ __forceinline__ int je(int t) const { return t ? je1 : je0; }
};
__device__ __forceinline__ Item read_item(const int* w, int per, int W) {
  Item it;
  it.t0 = w[0]; it.req = w[1]; it.p0 = w[2]; it.ntok = w[3]; it.kvh = w[4];
  it.kb = W > 0 ? max(0, it.p0 - W + 1) : 0;
  it.ke = it.p0 + it.ntok;
  it.s0 = (it.kb / STEP_KEYS) * STEP_KEYS;
  it.steps = (it.ke - it.s0 + STEP_KEYS - 1) / STEP_KEYS;
  // tile 0: tokens [0, min(ntok, per)), never empty; tile 1: tokens [per, ntok)
  it.jb0 = 0;
  it.je0 = (it.p0 + min(it.ntok, per) - it.s0 + STEP_KEYS - 1) / STEP_KEYS;
  it.jb1 = it.je1 = 0;
  if (it.ntok > per) {
    const int kb_1 = W > 0 ? max(0, it.p0 + per - W + 1) : 0;
    it.jb1 = (kb_1 - it.s0) / STEP_KEYS;
    it.je1 = it.steps;
  }
  return it;
}

// ------------------------------------------------------------------------------------------- tcgen05
// Shared-memory operand descriptors, 128-byte swizzle: rows of 128 bytes in groups of eight.
__device__ __forceinline__ uint64_t desc_k_major(const void* p, uint32_t group_stride_bytes) {  // 8-row groups that far apart
  return (uint64_t)((smem_u32(p) & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(group_stride_bytes >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}
__device__ __forceinline__ uint64_t desc_mn_major(const void* p, uint32_t block_stride_bytes, uint32_t group_stride_bytes) {
  // rows of 64 contiguous N elements; groups of 8 K-rows group_stride apart, 64-element N blocks block_stride apart
  return (uint64_t)((smem_u32(p) & 0x3FFFFu) >> 4) | ((uint64_t)(block_stride_bytes >> 4) << 16) |
         ((uint64_t)(group_stride_bytes >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// One thread issues all MMAs of a tile, and what it computes between two of them bounds their
// rate (measured: 96 cycles per MMA with the operands worked out in between, 64 = the nominal rate
// of N = 128 without).  So every descriptor of a batch is made first, and the MMAs follow in one
// straight line.
//
// S = Q K^T over the head's NB column blocks of 64 elements: 4 x NB MMAs of 16 elements each
// (32 bytes = 2 descriptor units on); the next column block of Q is 16 KB = 1,024 units on, of K
// 1,024 bytes = 64 units.  The first MMA overwrites S.
__device__ __forceinline__ void umma_scores(uint32_t d, uint64_t q, uint64_t k, uint32_t idesc) {
  if constexpr (NB == 2) {
    asm volatile(
        "{\n\t.reg .pred p0, p1;\n\t.reg .b64 a<8>, b<8>;\n\t"
        "setp.ne.b32 p0, 0, 0;\n\tsetp.eq.b32 p1, 0, 0;\n\t"
        "add.s64 a1, %1, 2;\n\tadd.s64 a2, %1, 4;\n\tadd.s64 a3, %1, 6;\n\t"
        "add.s64 a4, %1, 1024;\n\tadd.s64 a5, %1, 1026;\n\tadd.s64 a6, %1, 1028;\n\tadd.s64 a7, %1, 1030;\n\t"
        "add.s64 b1, %2, 2;\n\tadd.s64 b2, %2, 4;\n\tadd.s64 b3, %2, 6;\n\t"
        "add.s64 b4, %2, 64;\n\tadd.s64 b5, %2, 66;\n\tadd.s64 b6, %2, 68;\n\tadd.s64 b7, %2, 70;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %3, p1;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a2, b2, %3, p1;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a3, b3, %3, p1;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a4, b4, %3, p1;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a5, b5, %3, p1;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a6, b6, %3, p1;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a7, b7, %3, p1;\n\t}" ::"r"(d),
        "l"(q), "l"(k), "r"(idesc)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p0, p1;\n\t.reg .b64 a<4>, b<4>;\n\t"
        "setp.ne.b32 p0, 0, 0;\n\tsetp.eq.b32 p1, 0, 0;\n\t"
        "add.s64 a1, %1, 2;\n\tadd.s64 a2, %1, 4;\n\tadd.s64 a3, %1, 6;\n\t"
        "add.s64 b1, %2, 2;\n\tadd.s64 b2, %2, 4;\n\tadd.s64 b3, %2, 6;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %3, p1;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a2, b2, %3, p1;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a3, b3, %3, p1;\n\t}" ::"r"(d),
        "l"(q), "l"(k), "r"(idesc)
        : "memory");
  }
}
// O (+)= P V over the step's 128 keys: 8 MMAs of 16 keys each; P (in tensor memory) moves on by 8
// columns, V's descriptor by two row groups = 2 x NB x 1,024 bytes = NB x 128 units.
__device__ __forceinline__ void umma_product(uint32_t d, uint32_t p, uint64_t v, uint32_t idesc, uint32_t accumulate_first) {
  asm volatile(
      "{\n\t.reg .pred p0, p1;\n\t.reg .b32 a<8>;\n\t.reg .b64 b<8>;\n\t"
      "setp.ne.b32 p0, %4, 0;\n\tsetp.eq.b32 p1, 0, 0;\n\t"
      "add.u32 a1, %1, 8;\n\tadd.u32 a2, %1, 16;\n\tadd.u32 a3, %1, 24;\n\tadd.u32 a4, %1, 32;\n\t"
      "add.u32 a5, %1, 40;\n\tadd.u32 a6, %1, 48;\n\tadd.u32 a7, %1, 56;\n\t"
      "add.s64 b1, %2, %5;\n\tadd.s64 b2, %2, %6;\n\tadd.s64 b3, %2, %7;\n\tadd.s64 b4, %2, %8;\n\t"
      "add.s64 b5, %2, %9;\n\tadd.s64 b6, %2, %10;\n\tadd.s64 b7, %2, %11;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], b1, %3, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a2], b2, %3, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a3], b3, %3, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a4], b4, %3, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a5], b5, %3, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a6], b6, %3, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a7], b7, %3, p1;\n\t}" ::"r"(d),
      "r"(p), "l"(v), "r"(idesc), "r"(accumulate_first), "n"(NB * 128), "n"(2 * NB * 128), "n"(3 * NB * 128), "n"(4 * NB * 128),
      "n"(5 * NB * 128), "n"(6 * NB * 128), "n"(7 * NB * 128)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
                   smem_u32(dst)),
               "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, float* v) {  // tmem_ld_wait() before v is read
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,"
      "%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  tmem_ld32_issue(taddr, v);
  tmem_ld_wait();
}
__device__ __forceinline__ float fast_exp2(float x) {  // 2^x, -inf -> 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Two float32 operations in one instruction (sm_100): a softmax warp is bound by the number of
// instructions it can issue, and the scaling and the sums of a row are half as many this way.
__device__ __forceinline__ void fma2(float& d0, float& d1, float a0, float a1, float b, float c) {  // d = a * b + c, twice
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tmov.b64 rc, {%5, %5};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
__device__ __forceinline__ void add2(float& d0, float& d1, float a0, float a1) {  // d += a, twice
  asm("{\n\t.reg .b64 ra, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rd, {%0, %1};\n\t"
      "add.rn.f32x2 rd, rd, ra;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "+f"(d0), "+f"(d1)
      : "f"(a0), "f"(a1));
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {  // one instruction on sm_100
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ void tmem_st32_words(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
      "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31};" ::"r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
      "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]),
      "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]),
      "r"(v[30]), "r"(v[31]), "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16_words(uint32_t taddr, uint32_t* r) {  // waits for the data
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16_words(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15};" ::"r"(v[0]), "r"(v[1]),
      "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]),
      "r"(v[14]), "r"(v[15]), "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ------------------------------------------------------------------------------------------- producers
// One warp streams one side (keys or values) of an item: stage after stage of 128 keys of the
// request whose block table is `table`, restricted to [kb, ke).  A piece is the rows of one page
// that fall into the stage (at most 16 pieces: pages of 8 keys or more); lane i brings piece i,
// in whole row groups of 8 (rows of a group that lie outside [kb, ke) come along: the consumers
// mask them and clear their values).  Pages that were given back are not copied.  Everything that
// does not need the stage itself (page lookup, addresses, byte counts) is done before the wait for
// the stage to be free.  Returns false when a wait gave up.
__device__ __forceinline__ bool stream_side(const __nv_bfloat16* cache, const int* table, const Item& it, int nkv, int ps,
                                            __nv_bfloat16* ring, uint64_t* full, uint64_t* empty, int& count,
                                            volatile int* abort_flag, int* status, int lane, int trace_role) {
  const int piece = ps % 64 == 0 ? 64 : ps % 32 == 0 ? 32 : ps % 16 == 0 ? 16 : ps;  // divides the page and the stage
  const int pieces = STEP_KEYS / piece;
  const int ps_shift = (ps & (ps - 1)) == 0 ? __ffs(ps) - 1 : -1;
  const long long tile_elems = (long long)ps * HD, page_elems = tile_elems * nkv, head_off = (long long)it.kvh * tile_elems;
  for (int j = 0; j < it.steps; ++j, ++count) {
    const int slot = count % KV_STAGES;
    const int base = it.s0 + j * STEP_KEYS;
    const int kp = base + lane * piece;
    const bool inside = base >= it.kb && base + STEP_KEYS <= it.ke;  // every row of the stage is wanted
    const bool mine = lane < pieces && kp < it.ke && kp + piece > it.kb;
    int page = -1;
    if (mine) {
      page = table[ps_shift >= 0 ? kp >> ps_shift : kp / ps];
      if (page < 0) atomicExch(status, STATUS_BAD_PAGE);
    }
    int lo = 0, hi = 0;
    if (page >= 0) {
      lo = max(0, it.kb - kp) & ~7;
      hi = (min(piece, it.ke - kp) + 7) & ~7;
    }
    const int n = hi - lo;
    uint32_t bytes = (uint32_t)STAGE_BYTES_1;
    if (!inside || __any_sync(0xffffffffu, mine && page < 0)) {
      bytes = (uint32_t)n * HD * 2u;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) bytes += __shfl_xor_sync(0xffffffffu, bytes, o);
    }
    const int r0 = (ps_shift >= 0 ? kp & (ps - 1) : kp % ps) + lo, i0 = kp - base + lo;  // first row in the page, in the stage
    const __nv_bfloat16* src = cache + (long long)page * page_elems + head_off + (long long)r0 * HD;
    __nv_bfloat16* dst = ring + (size_t)slot * STAGE_ELEMS_1 + i0 * HD;
    // all lanes leave together or not at all
    if (count >= KV_STAGES && !__all_sync(0xffffffffu, mbar_wait(empty + slot, ((count / KV_STAGES) & 1) ^ 1, abort_flag, status)))
      return false;
    if (lane == 0) mbar_arrive_expect_tx(full + slot, bytes);
    __syncwarp();
    if (n > 0) bulk_load(dst, src, n * HD * 2, full + slot);
    if (lane == 0) TRACE(trace_role, count, 0);
  }
  return true;
}

// ------------------------------------------------------------------------------------------- kernel
__global__ void __launch_bounds__(THREADS, 1) attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const PrefillArgs a) {
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
  unsigned char* q_mem = smem;                                                       // [2 tiles][column block][128 rows][128 bytes]
  __nv_bfloat16* k_ring = reinterpret_cast<__nv_bfloat16*>(smem + 2 * Q_BYTES);       // [KV_STAGES][128 keys]
  __nv_bfloat16* v_ring = k_ring + (size_t)KV_STAGES * STAGE_ELEMS_1;
  uint64_t* k_full = reinterpret_cast<uint64_t*>(v_ring + (size_t)KV_STAGES * STAGE_ELEMS_1);
  uint64_t* k_empty = k_full + KV_STAGES;
  uint64_t* v_full = k_empty + KV_STAGES;
  uint64_t* v_empty = v_full + KV_STAGES;
  uint64_t* q_full = v_empty + KV_STAGES;  // [2] each of the following: one per tile
  uint64_t* q_empty = q_full + 2;          // the tile's last S of an item has read Q
  uint64_t* s_full = q_empty + 2;
  uint64_t* p_full = s_full + 2;
  uint64_t* o_ready = p_full + 2;          // the tile's last product of an item has completed
  uint64_t* o_free = o_ready + 2;          // the tile's output has been read out of tensor memory
  uint64_t* turn = o_free + 2;             // [2][4]: whose turn it is on a scheduler's special-function unit
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(turn + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = a.nh / a.nkv, per = BM / G, ps = a.page_size, W = a.window;
  const int* my_work = a.work + (size_t)blockIdx.x * WORK_INTS;
  const size_t work_step = (size_t)gridDim.x * WORK_INTS;

  if (tid == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(k_full + s, 1); mbar_init(k_empty + s, 2);
      mbar_init(v_full + s, 1); mbar_init(v_empty + s, 2);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(q_full + t, 1); mbar_init(q_empty + t, 1);
      mbar_init(s_full + t, 1); mbar_init(p_full + t, 4);
      mbar_init(o_ready + t, 1); mbar_init(o_free + t, 4);
    }
    for (int i = 0; i < 8; ++i) mbar_init(turn + i, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // Only now may the kernel behind this one become resident: it may hold tensor memory while it
  // waits for this grid to end, so every block of this grid must have its own columns first.
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t tmem_base = *tmem_slot;

  if (warp >= SOFTMAX_WARPS) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS_OTHER));
    if (warp == K_WARP) {
      // ------------------------------------------------------------------ query tiles and keys
      int count = 0, loads[2] = {0, 0};
      for (int k = 0; k < a.queue_len; ++k) {
        const Item it = read_item(my_work + k * work_step, per, W);
        if (it.ntok <= 0) break;
        bool ok = true;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (it.je(t) <= it.jb(t)) continue;
          if (loads[t] > 0) ok = ok && __all_sync(0xffffffffu, mbar_wait(q_empty + t, (loads[t] - 1) & 1, abort_flag, a.status));
          if (!ok) break;
          if (lane == 0) {
            mbar_arrive_expect_tx(q_full + t, (uint32_t)(NB * 64 * G * per * 2));
#pragma unroll
            for (int b = 0; b < NB; ++b)
              tma_load_3d(q_mem + t * Q_BYTES + b * (BM * 128), &map_q, b * 64, it.kvh * G, it.t0 + t * per, q_full + t);
          }
          ++loads[t];
        }
        if (!ok) break;
        if (!stream_side(a.k_cache, a.block_table + (size_t)it.req * a.table_stride, it, a.nkv, ps, k_ring, k_full, k_empty, count,
                         abort_flag, a.status, lane, 4))
          break;
      }
    } else if (warp == V_WARP) {
      // ------------------------------------------------------------------ values
      int count = 0;
      for (int k = 0; k < a.queue_len; ++k) {
        const Item it = read_item(my_work + k * work_step, per, W);
        if (it.ntok <= 0) break;
        if (!stream_side(a.v_cache, a.block_table + (size_t)it.req * a.table_stride, it, a.nkv, ps, v_ring, v_full, v_empty, count,
                         abort_flag, a.status, lane, 5))
          break;
      }
    } else if (lane == 0) {
      // ------------------------------------------------------------------ the MMAs of one tile
      const int t = warp - ISSUE_WARP;
      const uint32_t tmem_s = tmem_base + (uint32_t)(TMEM_S + t * TMEM_TILE), tmem_o = tmem_base + (uint32_t)(TMEM_O + t * TMEM_TILE);
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(STEP_KEYS >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      const uint64_t qd = desc_k_major(q_mem + t * Q_BYTES, 1024);
      int count = 0, steps_done = 0, items_done = 0;  // stages before this item; steps and items in which this tile took part
      bool ok = true;
      for (int k = 0; k < a.queue_len && ok; ++k) {
        const Item it = read_item(my_work + k * work_step, per, W);
        if (it.ntok <= 0) break;
        const int jb = it.jb(t), je = it.je(t);
        // round i: the product of step i - 1, then at once the scores of step i
        for (int i = 0; i <= it.steps && ok; ++i) {
          const int jp = i - 1;
          if (jp >= 0) {
            const int slot = (count + jp) % KV_STAGES;
            const uint32_t stage_phase = ((count + jp) / KV_STAGES) & 1;
            if (jp < jb || jp >= je) {  // a step of the other tile only: hand its values on
              ok = mbar_wait(v_full + slot, stage_phase, abort_flag, a.status);
              if (ok) mbar_arrive(v_empty + slot);
            } else {
              // everything the batch needs is made ready first; the softmax's hand-over is waited for last
              const uint64_t vd = desc_mn_major(v_ring + (size_t)slot * STAGE_ELEMS_1, 1024, NB * 1024);
              ok = mbar_wait(v_full + slot, stage_phase, abort_flag, a.status);
              // the first product of an item overwrites O: the item before must have been read out
              if (jp == jb && items_done > 0) ok = ok && mbar_wait(o_free + t, (items_done - 1) & 1, abort_flag, a.status);
              const bool more = i < je;  // the scores of step i follow at once
              uint64_t kd = 0;
              if (more) {
                const int kslot = (count + i) % KV_STAGES;
                kd = desc_k_major(k_ring + (size_t)kslot * STAGE_ELEMS_1, NB * 1024);
                ok = ok && mbar_wait(k_full + kslot, ((count + i) / KV_STAGES) & 1, abort_flag, a.status);
              }
              ok = ok && mbar_wait(p_full + t, steps_done & 1, abort_flag, a.status);
              if (!ok) break;
              tc_fence_after();
              TRACE(t, count + jp, 2);
              umma_product(tmem_o, tmem_s, vd, idesc_o, jp > jb ? 1u : 0u);
              // S overwrites the probabilities: the product that reads them was issued just above
              if (more) umma_scores(tmem_s, qd, kd, idesc_s);
              TRACE(t, count + jp, 3);
              umma_commit(v_empty + slot);
              if (jp == je - 1) umma_commit(o_ready + t);
              ++steps_done;
              if (more) {
                umma_commit(s_full + t);
                umma_commit(k_empty + (count + i) % KV_STAGES);
                if (i == je - 1) umma_commit(q_empty + t);
              }
            }
          }
          if (i < it.steps && ok) {
            const int slot = (count + i) % KV_STAGES;
            const uint32_t stage_phase = ((count + i) / KV_STAGES) & 1;
            if (i < jb || i >= je) {
              ok = mbar_wait(k_full + slot, stage_phase, abort_flag, a.status);
              if (ok) mbar_arrive(k_empty + slot);
            } else if (i == jb) {  // the first scores of an item (the later ones follow their step's product above)
              ok = mbar_wait(q_full + t, items_done & 1, abort_flag, a.status);
              ok = ok && mbar_wait(k_full + slot, stage_phase, abort_flag, a.status);
              if (!ok) break;
              tc_fence_after();
              TRACE(t, count + i, 0);
              umma_scores(tmem_s, qd, desc_k_major(k_ring + (size_t)slot * STAGE_ELEMS_1, NB * 1024), idesc_s);
              umma_commit(s_full + t);
              umma_commit(k_empty + slot);
              if (i == je - 1) umma_commit(q_empty + t);
              TRACE(t, count + i, 1);
            }
          }
        }
        count += it.steps;
        if (je > jb) ++items_done;
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax: one row per thread, one tile per four warps
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS_SOFTMAX));
    const int t = warp >> 2, quarter = warp & 3;
    const int row = quarter * 32 + lane;  // = lane of tensor memory
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t tmem_s = tmem_base + lane_base + (uint32_t)(TMEM_S + t * TMEM_TILE);
    const uint32_t tmem_o = tmem_base + lane_base + (uint32_t)(TMEM_O + t * TMEM_TILE);
    // The exponentials of a step are what the special-function unit of a scheduler is busy with for
    // as long as the tensor cores are with the step's MMAs, and a scheduler has one warp of each
    // tile.  Left alone, the two tiles fall into step (both wait for the same keys): both
    // exponentiate, then both multiply, and each unit idles half of the time.  So the two warps
    // of a scheduler take turns, step by step, tile 0 first: a warp exponentiates only when the
    // other has finished the same step's turn (or had nothing to do in it).
    uint64_t* my_turn = turn + t * 4 + quarter;        // completes once per step when the other warp has passed
    uint64_t* other_turn = turn + (t ^ 1) * 4 + quarter;
    int count = 0, steps_done = 0, items_done = 0;
    bool ok = true;
    for (int k = 0; k < a.queue_len && ok; ++k) {
      const Item it = read_item(my_work + k * work_step, per, W);
      if (it.ntok <= 0) break;
      const int tl = t * per + row / G;
      const bool live = row < per * G && tl < it.ntok;
      const int qpos = it.p0 + min(tl, it.ntok - 1);
      const int lo = W > 0 ? max(0, qpos - W + 1) : 0;
      float m_ref = -INFINITY, l = 0.f;  // the row's reference maximum (in units of log2) and its sum against it
      for (int j = 0; j < it.steps; ++j, ++count) {
        if (j < it.jb(t) || j >= it.je(t)) {  // nothing of this tile in the step: pass the turn on
          if (t == 1 || count > 0) ok = __all_sync(0xffffffffu, mbar_wait(my_turn, (t == 1 ? count : count - 1) & 1, abort_flag, a.status));
          if (!ok) break;
          if (lane == 0) mbar_arrive(other_turn);
          continue;
        }
        const int base = it.s0 + j * STEP_KEYS;
        // every give-up below is taken by the whole warp or by none of it: the tensor-memory
        // instructions and __syncwarp that follow a wait want all 32 lanes
        ok = __all_sync(0xffffffffu, mbar_wait(s_full + t, steps_done & 1, abort_flag, a.status));
        if (!ok) break;
        tc_fence_after();
        if (tid % 128 == 0) TRACE(2 + t, count, 0);
        float s[STEP_KEYS];
#pragma unroll
        for (int c0 = 0; c0 < STEP_KEYS; c0 += 32) tmem_ld32_issue(tmem_s + c0, s + c0);
        tmem_ld_wait();
        if (tid % 128 == 0) TRACE(2 + t, count, 1);
        if (base + STEP_KEYS - 1 > qpos || base < lo) {  // a block at the causal or the window's edge
#pragma unroll
          for (int c = 0; c < STEP_KEYS; ++c)
            if (base + c > qpos || base + c < lo) s[c] = -INFINITY;
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < STEP_KEYS; c += 8) {
          mx4[0] = fmax3(mx4[0], s[c], s[c + 1]);
          mx4[1] = fmax3(mx4[1], s[c + 2], s[c + 3]);
          mx4[2] = fmax3(mx4[2], s[c + 4], s[c + 5]);
          mx4[3] = fmax3(mx4[3], s[c + 6], s[c + 7]);
        }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * a.scale_log2;  // the scale is positive
        // move the reference only when it pays (any row of the warp: the tensor-memory instructions
        // below are executed by whole warps)
        const bool warp_need = __any_sync(0xffffffffu, mx > m_ref + RESCALE_AT);
        if (warp_need) {
          const float m_new = fmaxf(m_ref, mx);
          const float corr = m_ref == -INFINITY ? 0.f : exp2f(m_ref - m_new);
          l *= corr;
          m_ref = m_new;
          if (j > it.jb(t)) {  // this step's S was issued behind the product of the step before and has completed: O is at rest
#pragma unroll 1
            for (int c0 = 0; c0 < HD; c0 += 16) {  // sixteen columns at a time: the row of scores stays in registers meanwhile
              uint32_t w[16];
              tmem_ld16_words(tmem_o + c0, w);
#pragma unroll
              for (int c = 0; c < 16; ++c) w[c] = __float_as_uint(__uint_as_float(w[c]) * corr);
              tmem_st16_words(tmem_o + c0, w);
            }
          }
        }
        const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;
        if (tid % 128 == 0) TRACE(2 + t, count, 2);
        if (t == 1 || count > 0) ok = __all_sync(0xffffffffu, mbar_wait(my_turn, (t == 1 ? count : count - 1) & 1, abort_flag, a.status));
        if (!ok) break;
        if (tid % 128 == 0) TRACE(2 + t, count, 3);
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int h = 0; h < 4; ++h) {  // 32 keys = 16 columns of P at a time, over the columns of S that are in registers already
          // the exponentials of a chunk stand in one straight line: the special-function unit takes one
          // every eight cycles, and the scaling before and the sums and conversions after fit in between
          float e[32];
#pragma unroll
          for (int c = 0; c < 32; c += 2) fma2(e[c], e[c + 1], s[h * 32 + c], s[h * 32 + c + 1], a.scale_log2, neg_m);
#pragma unroll
          for (int c = 0; c < 32; ++c) asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(e[c]) : "f"(e[c]));
          uint32_t pw[16];
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            add2(sum4[c & 3], sum4[(c & 3) + 1], e[c], e[c + 1]);
            pw[c >> 1] = pack_bf16(e[c], e[c + 1]);
          }
          tmem_st16_words(tmem_s + h * 16, pw);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(other_turn);
        if (tid % 128 == 0) TRACE(2 + t, count, 4);
        l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
        if (base < it.kb || base + STEP_KEYS > it.ke) {
          // an edge stage: value rows of keys outside [kb, ke) get zero weights, but must not hold NaN
          // patterns (they were not copied, or came along with their row group): this warp clears its quarter
          ok = __all_sync(0xffffffffu, mbar_wait(v_full + count % KV_STAGES, (count / KV_STAGES) & 1, abort_flag, a.status));
          if (!ok) break;
          unsigned char* vs = reinterpret_cast<unsigned char*>(v_ring + (size_t)(count % KV_STAGES) * STAGE_ELEMS_1);
          for (int i = lane; i < 32 * NB * 8; i += 32) {
            const int r = quarter * 32 + i / (NB * 8), bc = i % (NB * 8);
            if (base + r < it.kb || base + r >= it.ke)
              *reinterpret_cast<uint4*>(vs + ((r >> 3) * NB + (bc >> 3)) * 1024 + (r & 7) * 128 + ((bc & 7) << 4)) = make_uint4(0, 0, 0, 0);
          }
          fence_proxy_async();  // the cleared rows are read by the tensor cores through the async proxy
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full + t);
        if (tid % 128 == 0) TRACE(2 + t, count, 5);
        ++steps_done;
      }
      if (!ok) break;
      if (it.je(t) <= it.jb(t)) continue;
      // ---------------------------------------------------------------- the item's output rows
      ok = __all_sync(0xffffffffu, mbar_wait(o_ready + t, items_done & 1, abort_flag, a.status));
      if (!ok) break;
      ++items_done;
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = a.out + (size_t)(it.t0 + tl) * a.nh * HD + (size_t)(it.kvh * G + row % G) * HD;
#pragma unroll
      for (int c0 = 0; c0 < HD; c0 += 32) {
        float o[32];
        tmem_ld32(tmem_o + c0, o);
        if (live) {
#pragma unroll
          for (int c = 0; c < 32; c += 8)
            *reinterpret_cast<uint4*>(dst + c0 + c) = make_uint4(pack_bf16(o[c] * inv, o[c + 1] * inv), pack_bf16(o[c + 2] * inv, o[c + 3] * inv),
                                                                 pack_bf16(o[c + 4] * inv, o[c + 5] * inv), pack_bf16(o[c + 6] * inv, o[c + 7] * inv));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_free + t);
    }
  }
  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) for (int i = 0; i < 2000; ++i) __nanosleep(100);  // let copies in flight land
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

constexpr size_t smem_bytes() { return 1024 + 2 * (size_t)Q_BYTES + 2 * (size_t)KV_STAGES * STAGE_BYTES_1 + (4 * KV_STAGES + 20) * 8 + 16; }

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiled encode_tiled() {
  static EncodeTiled fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiled>(p);
  }
  return fn;
}

// The query heads of [T, q_stride] rows as (64 elements of a head, heads of the group, tokens):
// a box is one column block of a query tile, rows in the order (token, head of the group), with
// the 128-byte swizzle; tokens beyond T read as zeros.
static int make_q_map(CUtensorMap* map, const void* q, long long T, int q_stride, int nh, int G, int per) {
  EncodeTiled enc = encode_tiled();
  if (!enc) return TB_ERR_BAD_SIZE;
  const cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)nh, (cuuint64_t)T};
  const cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)q_stride * 2};
  const cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)per};
  const cuuint32_t elem[3] = {1, 1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, elem,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 20000 + (int)r;
}

}  // namespace tb

extern "C" {

#ifdef TB_PF_TRACE
int tb_attention_prefill_tc_trace(long long* host) { return (int)cudaMemcpyFromSymbol(host, tb::tb_trace, sizeof(tb::tb_trace)); }
#endif
int tb_attention_prefill_tc_tile_rows() { return tb::BM; }
int tb_attention_prefill_tc_work_ints() { return tb::WORK_INTS; }

// work: [queue_len, blocks, 5] int32 on the device (first token row, request, first position, number of
// tokens (at most 2 * (128 / G)), kv head; no tokens = the block's queue has ended); grid = blocks.
// q: the [T, q_stride] rows whose first nh * hd columns are the query heads.  Pages of 8 keys or a multiple of 16.
int tb_attention_prefill_tc(void* stream, const void* q, int T, int q_stride, const void* k_cache, const void* v_cache,
                            const int* block_table, int table_stride, const int* work, int queue_len, int blocks, void* out,
                            int* status, int nh, int nkv, int page_size, int window, float scale) {
  if (queue_len <= 0 || blocks <= 0 || T <= 0) return 0;
  if (nkv <= 0 || nh % nkv != 0 || nh / nkv > tb::BM || !(scale > 0.f)) return TB_ERR_BAD_SIZE;
  if (!(page_size == 8 || (page_size > 0 && page_size % 16 == 0))) return TB_ERR_BAD_SIZE;
  if (((uintptr_t)q & 15) || (q_stride % 8) != 0) return TB_ERR_BAD_SIZE;
  const int G = nh / nkv, per = tb::BM / G;
  CUtensorMap map_q;
  const int e = tb::make_q_map(&map_q, q, T, q_stride, nh, G, per);
  if (e) return e;
  tb::PrefillArgs a;
  a.k_cache = (const __nv_bfloat16*)k_cache; a.v_cache = (const __nv_bfloat16*)v_cache;
  a.block_table = block_table; a.table_stride = table_stride;
  a.work = work; a.queue_len = queue_len; a.out = (__nv_bfloat16*)out; a.status = status;
  a.nh = nh; a.nkv = nkv; a.page_size = page_size; a.window = window;
  a.scale_log2 = scale * 1.4426950408889634f;
  static bool configured = false;
  const size_t smem = tb::smem_bytes();
  if (!configured) {
    cudaError_t ce = cudaFuncSetAttribute(tb::attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (ce != cudaSuccess) return (int)ce;
    configured = true;
  }
  return tb::launch(tb::attention_prefill_tc_kernel, dim3(blocks), dim3(tb::THREADS), smem, stream, map_q, a);
}

}  // extern "C"

// Host side of the prefill ops: upload -> (cast) -> one kernel launch -> download.
#include <cmath>
#include <string>

#include "grilly/ops/attention.h"
#include "grilly/ops/rope.h"

namespace grilly {
namespace ops {

namespace {
struct Scoped {   // releases pooled buffers on every exit path
    BufferPool& pool;
    std::vector<GrillyBuffer*> bufs;
    explicit Scoped(BufferPool& p) : pool(p) {}
    ~Scoped() {
        for (auto* b : bufs) pool.release(*b);
    }
    GrillyBuffer& add(GrillyBuffer& b) {
        bufs.push_back(&b);
        return b;
    }
};
struct Recording {  // begin() now, leave the recording state on every exit path
    CommandBatch& batch;
    explicit Recording(CommandBatch& b) : batch(b) { batch.begin(); }
    ~Recording() {
        if (batch.recording()) batch.submitNoWait();
    }
};
}  // namespace

void flashAttention2(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const float* Q, const float* K,
                     const float* V, const float* mask, float* output, uint32_t batchSize, uint32_t seqLen,
                     uint32_t numHeads, uint32_t headDim, float scale, uint32_t /*tileSizeQ*/,
                     uint32_t /*tileSizeK*/) {
    // tile sizes are accepted for signature compatibility; the kernel chooses its own tiling
    flashAttention2Ex(batch, pool, cache, Q, K, V, mask, output, batchSize, seqLen, numHeads, headDim, scale,
                      FlashAttention2Options{});
}

void flashAttention2Ex(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const float* Q, const float* K,
                       const float* V, const float* mask, float* output, uint32_t B, uint32_t S, uint32_t H,
                       uint32_t D, float scale, const FlashAttention2Options& opt) {
    if (!Q || !K || !V || !output) throw std::runtime_error("flashAttention2: null tensor pointer");
    if (B == 0 || S == 0 || H == 0 || D == 0) throw std::runtime_error("flashAttention2: empty shape");
    grl_device* dev = pool.device().handle();
    const size_t n = size_t(B) * H * S * D;
    const bool bf16 = opt.precision == Precision::BF16;
    if (bf16 && mask) throw std::runtime_error("flashAttention2: the bf16 path takes causal / seq_lens masks only");
    if (bf16 && D != 128) throw std::runtime_error("flashAttention2: the bf16 path needs head_dim 128");
    cache.getOrCreate(std::string(bf16 ? "flash-attention2-tcgen05/" : "flash-attention2/") + std::to_string(D));

    Scoped scope(pool);
    GrillyBuffer q32 = pool.acquire(n * 4), k32 = pool.acquire(n * 4), v32 = pool.acquire(n * 4),
                 out = pool.acquire(n * 4);
    scope.add(q32); scope.add(k32); scope.add(v32); scope.add(out);
    GrillyBuffer maskBuf, lensBuf, q16, k16, v16;
    scope.add(maskBuf); scope.add(lensBuf); scope.add(q16); scope.add(k16); scope.add(v16);

    Recording rec(batch);
    pool.upload(q32, Q, n * 4);
    pool.upload(k32, K, n * 4);
    pool.upload(v32, V, n * 4);

    grl_flash_params p{};
    p.q = q32.dptr; p.k = k32.dptr; p.v = v32.dptr; p.o = out.dptr;
    p.in_dtype = GRL_F32; p.out_dtype = GRL_F32;
    p.batch = int(B); p.heads = int(H); p.seq_len = int(S); p.head_dim = int(D);
    p.scale = scale;
    p.causal = opt.causal ? 1 : 0;
    p.rope_mode = int(opt.ropeMode); p.rope_theta = opt.ropeTheta; p.rope_scaling = opt.ropeScaling;
    p.kernel = GRL_KERNEL_AUTO;
    if (mask) {
        size_t mElems;
        if (opt.maskRank == 2) { mElems = size_t(B) * S; p.mask_kind = GRL_MASK_KEY; }
        else if (opt.maskRank == 3 || opt.maskBroadcastHeads) { mElems = size_t(B) * S * S; p.mask_kind = GRL_MASK_BSS; }
        else { mElems = size_t(B) * H * S * S; p.mask_kind = GRL_MASK_BHSS; }
        maskBuf = pool.acquire(mElems * 4);
        pool.upload(maskBuf, mask, mElems * 4);
        p.mask = static_cast<const float*>(maskBuf.dptr);
    }
    if (opt.seqLens) {
        lensBuf = pool.acquire(size_t(B) * 4);
        pool.upload(lensBuf, opt.seqLens, size_t(B) * 4);
        p.seq_lens = static_cast<const int32_t*>(lensBuf.dptr);
    }
    if (bf16) {
        q16 = pool.acquire(n * 2); k16 = pool.acquire(n * 2); v16 = pool.acquire(n * 2);
        check(grl_cast(dev, q32.dptr, GRL_F32, q16.dptr, GRL_BF16, n), "flashAttention2: cast");
        check(grl_cast(dev, k32.dptr, GRL_F32, k16.dptr, GRL_BF16, n), "flashAttention2: cast");
        check(grl_cast(dev, v32.dptr, GRL_F32, v16.dptr, GRL_BF16, n), "flashAttention2: cast");
        p.q = q16.dptr; p.k = k16.dptr; p.v = v16.dptr;
        p.in_dtype = GRL_BF16;
        p.kernel = GRL_KERNEL_TCGEN05;
    }
    check(grl_flash_fwd(dev, &p), "flashAttention2");
    check(grl_memcpy_d2h(dev, output, out.dptr, n * 4), "flashAttention2: download");
    batch.submit();
}

void flashAttention2Device(CommandBatch& /*batch*/, PipelineCache& cache, const GrillyBuffer& q, const GrillyBuffer& k,
                           const GrillyBuffer& v, GrillyBuffer& out, int inDtype, int outDtype, uint32_t B,
                           uint32_t S, uint32_t H, uint32_t D, float scale, bool causal,
                           const GrillyBuffer* seqLensDev, RopeMode ropeMode, float ropeTheta, float ropeScaling) {
    cache.getOrCreate("flash-attention2-device/" + std::to_string(D));
    grl_flash_params p{};
    p.q = q.dptr; p.k = k.dptr; p.v = v.dptr; p.o = out.dptr;
    p.in_dtype = inDtype; p.out_dtype = outDtype;
    p.batch = int(B); p.heads = int(H); p.seq_len = int(S); p.head_dim = int(D);
    p.scale = scale; p.causal = causal ? 1 : 0;
    p.seq_lens = seqLensDev && seqLensDev->dptr ? static_cast<const int32_t*>(seqLensDev->dptr) : nullptr;
    p.rope_mode = int(ropeMode); p.rope_theta = ropeTheta; p.rope_scaling = ropeScaling;
    p.kernel = GRL_KERNEL_AUTO;
    check(grl_flash_fwd(cache.device().handle(), &p), "flashAttention2Device");
}

void rope(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const float* x, float* y, uint32_t B,
          uint32_t S, uint32_t H, uint32_t D, float base, float scaling, RopeMode mode, const float* cosTable,
          const float* sinTable) {
    if (!x || !y) throw std::runtime_error("rope: null tensor pointer");
    if (mode == RopeMode::None) throw std::runtime_error("rope: mode must be Half or Interleaved");
    grl_device* dev = pool.device().handle();
    cache.getOrCreate("rope/" + std::to_string(D));
    const size_t n = size_t(B) * S * H * D, tn = size_t(S) * (D / 2);
    Scoped scope(pool);
    GrillyBuffer in = pool.acquire(n * 4), out = pool.acquire(n * 4), ct, st;
    scope.add(in); scope.add(out); scope.add(ct); scope.add(st);
    Recording rec(batch);
    pool.upload(in, x, n * 4);
    if (cosTable && sinTable) {
        ct = pool.acquire(tn * 4); st = pool.acquire(tn * 4);
        pool.upload(ct, cosTable, tn * 4);
        pool.upload(st, sinTable, tn * 4);
    }
    check(grl_rope(dev, static_cast<const float*>(in.dptr), static_cast<float*>(out.dptr), int(B), int(S), int(H),
                   int(D), base, scaling, int(mode), static_cast<const float*>(ct.dptr),
                   static_cast<const float*>(st.dptr)),
          "rope");
    check(grl_memcpy_d2h(dev, y, out.dptr, n * 4), "rope: download");
    batch.submit();
}

void attentionMask(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, float* scores, const float* keyMask,
                   uint32_t B, uint32_t H, uint32_t S, bool causal, float maskValue) {
    if (!scores) throw std::runtime_error("attentionMask: null scores");
    if (!causal && !keyMask) throw std::runtime_error("attentionMask: a (batch, seq) mask is required unless causal");
    grl_device* dev = pool.device().handle();
    cache.getOrCreate("attention-mask");
    const size_t n = size_t(B) * H * S * S;
    Scoped scope(pool);
    GrillyBuffer sc = pool.acquire(n * 4), km;
    scope.add(sc); scope.add(km);
    Recording rec(batch);
    pool.upload(sc, scores, n * 4);
    if (!causal) {
        km = pool.acquire(size_t(B) * S * 4);
        pool.upload(km, keyMask, size_t(B) * S * 4);
    }
    check(grl_attention_mask(dev, static_cast<float*>(sc.dptr), static_cast<const float*>(km.dptr), int(B), int(H),
                             int(S), causal ? 1 : 0, maskValue),
          "attentionMask");
    check(grl_memcpy_d2h(dev, scores, sc.dptr, n * 4), "attentionMask: download");
    batch.submit();
}

}  // namespace ops
}  // namespace grilly

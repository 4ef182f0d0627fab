// Host side of the prefill ops: upload -> (cast) -> one kernel launch -> download.
#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <mutex>
#include <cstdlib>
#include <exception>
#include <string>
#include <vector>

#include "grilly/host_workers.h"
#include "grilly/ops/attention.h"
#include "grilly/ops/rope.h"

namespace grilly {
namespace ops {

namespace {
constexpr size_t kPipelineMinBytes = 8u << 20;     // per tensor: below this one upload / launch / download
constexpr size_t kPipelineChunkBytes = 32u << 20;      // per tensor: the large chunks
constexpr size_t kPipelineHostCastPct = 100;   // all of it: with pinned sources 75 % was 5 % faster (16 host threads, 55 GB/s
                                              // link), but a pageable float32 source uploads synchronously and three times slower
constexpr size_t kPipelineLastChunkBytes = 4u << 20;   // per tensor: the last chunk (nothing hides its kernel and download)
struct Scoped {   // releases pooled buffers on every exit path
    BufferPool& pool;
    std::vector<GrillyBuffer*> bufs;
    explicit Scoped(BufferPool& p) : pool(p) {}
    ~Scoped() {
        // leaving through an exception: copies and kernels may still be in flight on the three queues
        if (std::uncaught_exceptions() > 0) pool.device().quiesce();
        for (auto* b : bufs) pool.release(*b);
    }
    GrillyBuffer& add(GrillyBuffer& b) {
        bufs.push_back(&b);
        return b;
    }
};
std::mutex g_infoMu;
PipelineInfo g_lastInfo;
std::atomic<bool> g_pipelineTiming{false};
// Measured by earlier calls of this process: what the host threads round per second (float32 bytes read) and
// what the link uploads per second.  They set the host-rounded share of a chunk when several processes share
// the host (one per GPU).
std::atomic<double> g_hostRoundBps{0.0}, g_linkBps{0.0};
double nowMs() {
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
struct Recording {  // begin() now, leave the recording state on every exit path
    CommandBatch& batch;
    explicit Recording(CommandBatch& b) : batch(b) { batch.begin(); }
    ~Recording() {
        if (batch.recording()) batch.submitNoWait();
    }
};
}  // namespace

PipelineInfo lastPipelineInfo() {
    std::lock_guard<std::mutex> lock(g_infoMu);
    return g_lastInfo;
}
void setPipelineTiming(bool on) { g_pipelineTiming.store(on); }

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
    if (bf16 && D != 128 && D != 64) throw std::runtime_error("flashAttention2: the bf16 path needs head_dim 128 or 64");
    cache.getOrCreate(std::string(bf16 ? "flash-attention2-tcgen05/" : "flash-attention2/") + std::to_string(D));

    Scoped scope(pool);
    const size_t slice = size_t(S) * D;                       // elements of one (b, h) slice
    const bool pipelined = n * 4 >= kPipelineMinBytes && (!mask || opt.maskRank == 2) && size_t(B) * H > 1;
    GrillyBuffer q32, k32, v32, out = pool.acquire(n * 4);
    // share of a chunk that the host threads round to bf16 themselves (the rest is cast on the device)
    size_t hostPct = kPipelineHostCastPct;
    // Per chunk the link is busy for ((1-x)*4 + x*2) bytes per element and the host threads for 4*x bytes per
    // element; the two overlap, so the best share x makes them equal: x = 2 r_h / (2 r_l + r_h) with the rounding
    // rate r_h and the link rate r_l this process measured in its earlier calls.  Measured on one B200 box (host
    // rounds at 59 GB/s, link at 45): 8.32 / 7.80 / 7.58 / 7.81 / 7.48 / 7.67 ms per call at 100 / 90 / 80 / 70 / 60 /
    // 40 %; the rule picks 79 %.  The first call has no measurement yet and rounds everything on the host.
    // Several processes of one node (one per GPU) share the host's cores and memory: their rounding threads
    // oversubscribe the cores and take memory bandwidth from the copies, which the two-rate model does not see.
    // Measured with 4 processes: 15.7 / 16.3 / 19.8 / 24.4 ms per call at 0 / 30 / 62 (the rule) / 100 %; with 8:
    // 26.8 / 27.7 / 27.4 at 0 / 15 / 33 %; with 2: 22.5 / 26.8 / 27.5 / 26.7 TFLOP/s in total at 100 / 50 / 25 / 0 %.
    // So a process that shares the host uploads float32 and casts on the device.
    {
        int lws = 1;
        if (const char* e = std::getenv("LOCAL_WORLD_SIZE")) lws = std::max(1, std::atoi(e));
        const double rh = g_hostRoundBps.load(), rl = g_linkBps.load();
        if (lws > 1) hostPct = 0;
        else if (rh > 0.0 && rl > 0.0) hostPct = size_t(std::min(100.0, std::max(0.0, 100.0 * 2.0 * rh / (2.0 * rl + rh))));
    }
    if (const char* e = std::getenv("GRILLY_PIPELINE_HOST_CAST_PCT")) hostPct = size_t(std::min(100, std::max(0, std::atoi(e))));
    if (!(pipelined && bf16 && hostPct == 100)) {
        q32 = pool.acquire(n * 4); k32 = pool.acquire(n * 4); v32 = pool.acquire(n * 4);
    }
    scope.add(q32); scope.add(k32); scope.add(v32); scope.add(out);
    GrillyBuffer maskBuf, lensBuf, q16, k16, v16;
    scope.add(maskBuf); scope.add(lensBuf); scope.add(q16); scope.add(k16); scope.add(v16);

    // Large calls are bound by the host link (4 tensors of n floats cross it), not by the kernel: cut the
    // (batch, head) slices into chunks and let the upload of chunk c+1, the kernel of chunk c and the
    // download of chunk c-1 run on three queues at once.  Heads are independent, so a chunk is a smaller
    // problem of the same kind.  Dense masks keep the one-shot path below.
    if (pipelined) {
        // Chunk plan, in (b, h) slices.  Every chunk boundary costs the upload queue a bubble (the event
        // between two copies), and the last chunk's kernel and download are not hidden by anything: so
        // few, large chunks first and a short geometric tail (… 32, 32, 16, 8, 4 MiB per tensor).
        size_t bigBytes = kPipelineChunkBytes, lastBytes = kPipelineLastChunkBytes;
        if (const char* e = std::getenv("GRILLY_PIPELINE_CHUNK_MB")) bigBytes = size_t(std::max(1, std::atoi(e))) << 20;
        if (const char* e = std::getenv("GRILLY_PIPELINE_LAST_MB")) lastBytes = size_t(std::max(1, std::atoi(e))) << 20;
        const size_t total = size_t(B) * H;
        const size_t big = std::max<size_t>(1, bigBytes / (slice * 4)), last = std::max<size_t>(1, lastBytes / (slice * 4));
        std::vector<size_t> plan;                      // built back to front
        for (size_t left = total, c = std::min(last, big); left > 0;) {
            const size_t take = std::min(c, left);
            plan.push_back(take);
            left -= take;
            c = std::min(big, c * 2);
        }
        std::reverse(plan.begin(), plan.end());
        const bool perBatch = mask || opt.seqLens;     // a chunk then stays inside one batch row
        grl_device* up = pool.device().uploadQueue();
        grl_device* down = pool.device().downloadQueue();
        struct Events {   // destroyed on every exit path
            std::vector<grl_event*> v;
            ~Events() { for (auto* e : v) grl_event_destroy(e); }
            grl_event* make(bool timed = false) {
                grl_event* e = nullptr;
                check(timed ? grl_event_create(&e) : grl_event_create_untimed(&e), "flashAttention2: event");
                v.push_back(e);
                return e;
            }
        } events;
        const bool timing = g_pipelineTiming.load();
        const double tCall = nowMs();
        PipelineInfo info;
        info.valid = true; info.timed = timing; info.hostCastPct = bf16 ? int(hostPct) : 0; info.chunks = int(plan.size());
        info.hostThreads = HostWorkers::instance().threads();
        std::vector<std::pair<grl_event*, grl_event*>> upSpans, mainSpans, downSpans;   // (begin, end) per chunk
        auto mark = [&](grl_device* q, bool on) -> grl_event* {
            if (!on) return nullptr;
            grl_event* e = events.make(true);
            check(grl_event_record(q, e), "flashAttention2: event");
            return e;
        };
        Recording rec(batch);
        if (mask) {
            maskBuf = pool.acquire(size_t(B) * S * 4);
            pool.upload(maskBuf, mask, size_t(B) * S * 4);
        }
        if (opt.seqLens) {
            lensBuf = pool.acquire(size_t(B) * 4);
            pool.upload(lensBuf, opt.seqLens, size_t(B) * 4);
        }
        if (bf16) { q16 = pool.acquire(n * 2); k16 = pool.acquire(n * 2); v16 = pool.acquire(n * 2); }
        // the buffers may have been used by earlier work on the main queue
        grl_event* start = events.make();
        check(grl_event_record(dev, start), "flashAttention2: event");
        check(grl_event_wait(up, start), "flashAttention2: event");
        check(grl_event_wait(down, start), "flashAttention2: event");
        auto at = [](const GrillyBuffer& b, size_t byteOff) { return static_cast<char*>(b.dptr) + byteOff; };
        size_t s0 = 0, chunkIndex = 0;
        grl_event* stagingBusy[2] = {nullptr, nullptr};
        for (size_t chunk : plan) {
            const size_t s1 = s0 + chunk;
            // upload the whole chunk, then launch it piece by piece (one piece unless it crosses a batch row)
            const size_t e0 = s0 * slice, ne = chunk * slice;
            // the upload queue is always timed (it feeds the share rule): one span per group of copies, so that the
            // time the queue sits idle while the host threads round is not counted as copy time
            if (bf16) {
                // Two routes share the chunk so that the host threads and the link finish together: the tail
                // of the chunk is uploaded as float32 (and cast on the device), the head is rounded to bf16 by
                // the host threads meanwhile -- half the bytes to upload -- into one of two pinned staging sets
                // (a set is reused only after the upload that read it has completed).
                const size_t nHost = chunk * hostPct / 100, eh = nHost * slice;     // slices / elements via the host
                const float* src[3] = {Q + e0, K + e0, V + e0};
                const GrillyBuffer* dst32[3] = {&q32, &k32, &v32};
                const GrillyBuffer* dst16[3] = {&q16, &k16, &v16};
                if (eh < ne) {
                    grl_event* b0 = mark(up, true);
                    for (int x = 0; x < 3; ++x)
                        check(grl_memcpy_h2d(up, at(*dst32[x], (e0 + eh) * 4), src[x] + eh, (ne - eh) * 4),
                              "flashAttention2: upload");
                    upSpans.emplace_back(b0, mark(up, true));
                }
                const int set = int(chunkIndex & 1);
                if (eh > 0) {
                    if (stagingBusy[set]) check(grl_event_sync(stagingBusy[set]), "flashAttention2: staging");
                    for (int x = 0; x < 3; ++x) {
                        auto* st = static_cast<uint16_t*>(pool.device().pinnedStaging(set * 3 + x, big * slice * 2));
                        const double t0 = nowMs();
                        convertF32ToBF16(src[x], st, eh);
                        info.hostRoundMs += nowMs() - t0;
                        info.hostRoundBytes += double(eh) * 4;
                        grl_event* b0 = mark(up, true);
                        check(grl_memcpy_h2d(up, at(*dst16[x], e0 * 2), st, eh * 2), "flashAttention2: upload");
                        upSpans.emplace_back(b0, mark(up, true));
                    }
                }
                stagingBusy[set] = events.make(true);
                check(grl_event_record(up, stagingBusy[set]), "flashAttention2: event");
                check(grl_event_wait(dev, stagingBusy[set]), "flashAttention2: event");
                info.h2dBytes += 3.0 * (double(ne - eh) * 4 + double(eh) * 2);
                if (eh < ne)
                    for (int x = 0; x < 3; ++x)
                        check(grl_cast(dev, at(*dst32[x], (e0 + eh) * 4), GRL_F32, at(*dst16[x], (e0 + eh) * 2), GRL_BF16,
                                       ne - eh),
                              "flashAttention2: cast");
            } else {
                grl_event* upBegin = mark(up, true);
                check(grl_memcpy_h2d(up, at(q32, e0 * 4), Q + e0, ne * 4), "flashAttention2: upload");
                check(grl_memcpy_h2d(up, at(k32, e0 * 4), K + e0, ne * 4), "flashAttention2: upload");
                check(grl_memcpy_h2d(up, at(v32, e0 * 4), V + e0, ne * 4), "flashAttention2: upload");
                grl_event* uploaded = events.make(true);
                check(grl_event_record(up, uploaded), "flashAttention2: event");
                check(grl_event_wait(dev, uploaded), "flashAttention2: event");
                upSpans.emplace_back(upBegin, uploaded);
                info.h2dBytes += 3.0 * double(ne) * 4;
            }
            ++chunkIndex;
            grl_event* mainBegin = mark(dev, timing);
            for (size_t p0 = s0; p0 < s1;) {
                const size_t b = p0 / H;
                const size_t p1 = perBatch ? std::min(s1, (b + 1) * size_t(H)) : s1;
                const size_t pe = p0 * slice;
                grl_flash_params p{};
                p.o = at(out, pe * 4);
                if (bf16) {
                    p.q = at(q16, pe * 2); p.k = at(k16, pe * 2); p.v = at(v16, pe * 2);
                    p.in_dtype = GRL_BF16; p.kernel = GRL_KERNEL_TCGEN05;
                } else {
                    p.q = at(q32, pe * 4); p.k = at(k32, pe * 4); p.v = at(v32, pe * 4);
                    p.in_dtype = GRL_F32; p.kernel = GRL_KERNEL_AUTO;
                }
                p.out_dtype = GRL_F32;
                p.batch = 1; p.heads = int(p1 - p0); p.seq_len = int(S); p.head_dim = int(D);
                p.scale = scale; p.causal = opt.causal ? 1 : 0;
                p.rope_mode = int(opt.ropeMode); p.rope_theta = opt.ropeTheta; p.rope_scaling = opt.ropeScaling;
                if (mask) { p.mask_kind = GRL_MASK_KEY; p.mask = static_cast<const float*>(maskBuf.dptr) + b * S; }
                if (opt.seqLens) p.seq_lens = static_cast<const int32_t*>(lensBuf.dptr) + b;
                check(grl_flash_fwd(dev, &p), "flashAttention2");
                p0 = p1;
            }
            grl_event* computed = events.make(timing);
            check(grl_event_record(dev, computed), "flashAttention2: event");
            check(grl_event_wait(down, computed), "flashAttention2: event");
            grl_event* downBegin = mark(down, timing);
            check(grl_memcpy_d2h(down, output + e0, at(out, e0 * 4), ne * 4), "flashAttention2: download");
            if (timing) {
                mainSpans.emplace_back(mainBegin, computed);
                downSpans.emplace_back(downBegin, mark(down, true));
            }
            info.d2hBytes += double(ne) * 4;
            s0 = s1;
        }
        // the main queue outlives the call: make it wait for the copies before its buffers are reused
        grl_event* done = events.make();
        check(grl_event_record(down, done), "flashAttention2: event");
        check(grl_event_wait(dev, done), "flashAttention2: event");
        batch.submit();      // waits for the main queue (and so for `done`), reports kernel failures
        info.totalMs = nowMs() - tCall;
        auto busy = [](const std::vector<std::pair<grl_event*, grl_event*>>& spans) {
            double total = 0;
            for (auto& s : spans) {
                float ms = 0;
                if (grl_event_elapsed_ms(s.first, s.second, &ms) == GRL_OK) total += ms;
            }
            return total;
        };
        info.h2dMs = busy(upSpans);
        info.kernelMs = busy(mainSpans);
        info.d2hMs = busy(downSpans);
        if (info.hostRoundMs > 0.05) g_hostRoundBps.store(info.hostRoundBytes / (info.hostRoundMs * 1e-3));
        if (info.h2dMs > 0.05) g_linkBps.store(info.h2dBytes / (info.h2dMs * 1e-3));
        {
            std::lock_guard<std::mutex> lock(g_infoMu);
            g_lastInfo = info;
        }
        return;
    }

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

size_t swizzledBufferSize(uint32_t B, uint32_t H, uint32_t S, uint32_t D, uint32_t W) {
    const size_t sp = (size_t(S) + W - 1) / W * W, dp = (size_t(D) + W - 1) / W * W;
    return size_t(B) * H * sp * dp * sizeof(float);
}

void swizzle(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const float* input, float* output, uint32_t B,
             uint32_t H, uint32_t S, uint32_t D, uint32_t W, bool reverse) {
    if (!input || !output) throw std::runtime_error("swizzle: null tensor pointer");
    if (B == 0 || H == 0 || S == 0 || D == 0 || W == 0) throw std::runtime_error("swizzle: empty shape");
    cache.getOrCreate("kv-swizzle");
    const size_t plain = size_t(B) * H * S * D * 4, swz = swizzledBufferSize(B, H, S, D, W);
    const size_t inBytes = reverse ? swz : plain, outBytes = reverse ? plain : swz;
    Scoped scope(pool);
    GrillyBuffer in = pool.acquire(inBytes), out = pool.acquire(outBytes);
    scope.add(in); scope.add(out);
    grl_device* dev = pool.device().handle();
    Recording rec(batch);
    pool.upload(in, input, inBytes);
    check(grl_swizzle_kv(dev, static_cast<const float*>(in.dptr), static_cast<float*>(out.dptr), int(B), int(H), int(S),
                         int(D), int(W), reverse ? 1 : 0),
          "swizzle");
    check(grl_memcpy_d2h(dev, output, out.dptr, outBytes), "swizzle: download");
    batch.submit();
}

void attentionScores(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const float* Q, const float* K,
                     float* scores, uint32_t B, uint32_t S, uint32_t H, uint32_t D, float scale) {
    if (!Q || !K || !scores) throw std::runtime_error("attentionScores: null tensor pointer");
    if (B == 0 || S == 0 || H == 0 || D == 0) throw std::runtime_error("attentionScores: empty shape");
    cache.getOrCreate("attention-scores");
    const size_t qBytes = size_t(B) * S * H * D * 4, sBytes = size_t(B) * H * S * S * 4;
    Scoped scope(pool);
    GrillyBuffer q = pool.acquire(qBytes), k = pool.acquire(qBytes), sc = pool.acquire(sBytes);
    scope.add(q); scope.add(k); scope.add(sc);
    grl_device* dev = pool.device().handle();
    Recording rec(batch);
    pool.upload(q, Q, qBytes);
    pool.upload(k, K, qBytes);
    check(grl_attention_scores(dev, static_cast<const float*>(q.dptr), static_cast<const float*>(k.dptr),
                               static_cast<float*>(sc.dptr), int(B), int(S), int(H), int(D), scale),
          "attentionScores");
    check(grl_memcpy_d2h(dev, scores, sc.dptr, sBytes), "attentionScores: download");
    batch.submit();
}

void softmax(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const float* input, float* output, size_t rows,
             uint32_t features) {
    if (!input || !output) throw std::runtime_error("softmax: null tensor pointer");
    if (rows == 0 || features == 0) throw std::runtime_error("softmax: empty shape");
    cache.getOrCreate("activation-softmax");
    const size_t bytes = rows * features * 4;
    Scoped scope(pool);
    GrillyBuffer in = pool.acquire(bytes), out = pool.acquire(bytes);
    scope.add(in); scope.add(out);
    grl_device* dev = pool.device().handle();
    Recording rec(batch);
    pool.upload(in, input, bytes);
    check(grl_softmax(dev, static_cast<const float*>(in.dptr), static_cast<float*>(out.dptr), rows, int(features)), "softmax");
    check(grl_memcpy_d2h(dev, output, out.dptr, bytes), "softmax: download");
    batch.submit();
}

void attentionOutput(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const float* weights, const float* V,
                     float* output, uint32_t B, uint32_t S, uint32_t H, uint32_t D, bool causal) {
    if (!weights || !V || !output) throw std::runtime_error("attentionOutput: null tensor pointer");
    if (B == 0 || S == 0 || H == 0 || D == 0) throw std::runtime_error("attentionOutput: empty shape");
    cache.getOrCreate(causal ? "attention-output-gpt" : "attention-output");
    const size_t vBytes = size_t(B) * S * H * D * 4, wBytes = size_t(B) * H * S * S * 4;
    Scoped scope(pool);
    GrillyBuffer w = pool.acquire(wBytes), v = pool.acquire(vBytes), o = pool.acquire(vBytes);
    scope.add(w); scope.add(v); scope.add(o);
    grl_device* dev = pool.device().handle();
    Recording rec(batch);
    pool.upload(w, weights, wBytes);
    pool.upload(v, V, vBytes);
    check(grl_attention_output(dev, static_cast<const float*>(w.dptr), static_cast<const float*>(v.dptr),
                               static_cast<float*>(o.dptr), int(B), int(S), int(H), int(D), causal ? 1 : 0),
          "attentionOutput");
    check(grl_memcpy_d2h(dev, output, o.dptr, vBytes), "attentionOutput: download");
    batch.submit();
}

void attentionBackward(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const float* gradOutput, const float* Q,
                       const float* K, const float* V, const float* attnWeights, float* gradQ, float* gradK, float* gradV,
                       uint32_t B, uint32_t H, uint32_t S, uint32_t D, float scale) {
    if (!gradOutput || !Q || !K || !V || !attnWeights || !gradQ || !gradK || !gradV)
        throw std::runtime_error("attentionBackward: null tensor pointer");
    if (B == 0 || S == 0 || H == 0 || D == 0) throw std::runtime_error("attentionBackward: empty shape");
    cache.getOrCreate("attention-backward");
    const size_t tBytes = size_t(B) * H * S * D * 4, aBytes = size_t(B) * H * S * S * 4;
    Scoped scope(pool);
    GrillyBuffer go = pool.acquire(tBytes), q = pool.acquire(tBytes), k = pool.acquire(tBytes), v = pool.acquire(tBytes),
                 a = pool.acquire(aBytes), scratch = pool.acquire(aBytes), gq = pool.acquire(tBytes), gk = pool.acquire(tBytes),
                 gv = pool.acquire(tBytes);
    for (GrillyBuffer* b : {&go, &q, &k, &v, &a, &scratch, &gq, &gk, &gv}) scope.add(*b);
    grl_device* dev = pool.device().handle();
    Recording rec(batch);
    pool.upload(go, gradOutput, tBytes);
    pool.upload(q, Q, tBytes);
    pool.upload(k, K, tBytes);
    pool.upload(v, V, tBytes);
    pool.upload(a, attnWeights, aBytes);
    auto f = [](const GrillyBuffer& b) { return static_cast<float*>(b.dptr); };
    check(grl_attention_backward(dev, f(go), f(q), f(k), f(v), f(a), f(gq), f(gk), f(gv), f(scratch), int(B), int(H), int(S),
                                 int(D), scale),
          "attentionBackward");
    check(grl_memcpy_d2h(dev, gradQ, gq.dptr, tBytes), "attentionBackward: download");
    check(grl_memcpy_d2h(dev, gradK, gk.dptr, tBytes), "attentionBackward: download");
    check(grl_memcpy_d2h(dev, gradV, gv.dptr, tBytes), "attentionBackward: download");
    batch.submit();
}

}  // namespace ops
}  // namespace grilly

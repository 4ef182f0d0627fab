// Host side of the linear projection: upload -> (cast) -> one kernel -> download.
#include <stdexcept>
#include <string>

#include "grilly/ops/linear.h"

namespace grilly {
namespace ops {

void linearEx(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const float* x, const float* weights,
              const float* bias, float* output, const LinearParams& p, Precision precision) {
    if (!x || !weights || !output) throw std::runtime_error("linear: null tensor pointer");
    if (p.batchSeq == 0 || p.inputDim == 0 || p.outputDim == 0) throw std::runtime_error("linear: empty shape");
    const bool bf16 = precision == Precision::BF16;
    if (bf16 && p.inputDim % 8 != 0) throw std::runtime_error("linear: the bf16 path needs input_dim to be a multiple of 8");
    grl_device* dev = pool.device().handle();
    cache.getOrCreate(std::string(bf16 ? "fnn-linear-tcgen05/" : "fnn-linear/") + std::to_string(p.inputDim));
    const size_t nx = size_t(p.batchSeq) * p.inputDim, nw = size_t(p.outputDim) * p.inputDim, ny = size_t(p.batchSeq) * p.outputDim;
    GrillyBuffer xb = pool.acquire(nx * 4), wb = pool.acquire(nw * 4), yb = pool.acquire(ny * 4), bb, x16, w16;
    auto releaseAll = [&]() {
        pool.release(xb); pool.release(wb); pool.release(yb); pool.release(bb); pool.release(x16); pool.release(w16);
    };
    try {
        batch.begin();
        pool.upload(xb, x, nx * 4);
        pool.upload(wb, weights, nw * 4);
        const float* biasDev = nullptr;
        if (p.hasBias && bias) {
            bb = pool.acquire(size_t(p.outputDim) * 4);
            pool.upload(bb, bias, size_t(p.outputDim) * 4);
            biasDev = static_cast<const float*>(bb.dptr);
        }
        if (bf16) {
            x16 = pool.acquire(nx * 2);
            w16 = pool.acquire(nw * 2);
            check(grl_cast(dev, xb.dptr, GRL_F32, x16.dptr, GRL_BF16, nx), "linear: cast");
            check(grl_cast(dev, wb.dptr, GRL_F32, w16.dptr, GRL_BF16, nw), "linear: cast");
            check(grl_linear(dev, x16.dptr, w16.dptr, biasDev, static_cast<float*>(yb.dptr), int(p.batchSeq), int(p.inputDim),
                             int(p.outputDim), GRL_BF16), "linear");
        } else {
            check(grl_linear(dev, xb.dptr, wb.dptr, biasDev, static_cast<float*>(yb.dptr), int(p.batchSeq), int(p.inputDim),
                             int(p.outputDim), GRL_F32), "linear");
        }
        check(grl_memcpy_d2h(dev, output, yb.dptr, ny * 4), "linear: download");
        batch.submit();
    } catch (...) {
        if (batch.recording()) batch.submitNoWait();
        pool.device().quiesce();   // nothing in flight may still touch the buffers released below
        releaseAll();
        throw;
    }
    releaseAll();
}

void linear(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const float* x, const float* weights,
            const float* bias, float* output, const LinearParams& p) {
    linearEx(batch, pool, cache, x, weights, bias, output, p, Precision::FP32);
}

void fusedQKVProjection(CommandBatch& batch, BufferPool& pool, PipelineCache& cache, const float* x, const float* wQKV,
                        const float* bQKV, float* output, uint32_t batchSeq, uint32_t hiddenDim, uint32_t numHeads,
                        uint32_t headDim, Precision precision) {
    LinearParams p{batchSeq, hiddenDim, 3 * numHeads * headDim, bQKV ? 1u : 0u};
    linearEx(batch, pool, cache, x, wQKV, bQKV, output, p, precision);
}

}  // namespace ops
}  // namespace grilly

// grilly_core: pybind11 module with the reference's names, keyword arguments and defaults for the
// attention / KV-cache subset (cpp/python/bindings.cpp:169-206, 416-462, 592-694 of the reference),
// plus additive keyword arguments for the fused masks, RoPE, the bf16 tensor-core path and decode.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <memory>
#include <optional>
#include <string>
#include <thread>
#include <vector>

#include "grilly/buffer_pool.h"
#include "grilly/command_batch.h"
#include "grilly/device.h"
#include "grilly/host_workers.h"
#include "grilly/ops/attention.h"
#include "grilly/experimental/fused_attention.h"
#include "grilly/ops/kv_cache.h"
#include "grilly/ops/linear.h"
#include "grilly/ops/sharded_decode.h"
#include "grilly/ops/rope.h"
#include "grilly/pipeline_cache.h"

namespace py = pybind11;
using namespace grilly;
using FArr = py::array_t<float, py::array::c_style | py::array::forcecast>;
using IArr = py::array_t<int32_t, py::array::c_style | py::array::forcecast>;

/// One object holding device -> pool -> cache -> batch, like the reference's GrillyCoreContext.
struct GrillyCoreContext {
    GrillyDevice device;
    BufferPool pool;
    PipelineCache cache;
    CommandBatch batch;
    bool shadersLoaded = false;
    GrillyCoreContext() : device(), pool(device), cache(device), batch(device) {}
    explicit GrillyCoreContext(int ordinal) : device(ordinal), pool(device), cache(device), batch(device) {}
    /// Kernels are compiled into the library; the call is kept so that callers written for the
    /// Vulkan backend keep working.
    void loadShaders(const std::string&) { shadersLoaded = true; }
};

using ContextPtr = std::shared_ptr<GrillyCoreContext>;

/// HBM-resident tensor (float32 or bf16) owned by a Device's buffer pool.  Ops that take DeviceTensors
/// run asynchronously on the device's stream: no host copy, no wait (Device.synchronize() waits).
struct DeviceTensor {
    ContextPtr ctx;
    GrillyBuffer buf;
    std::vector<py::ssize_t> shape;
    int dtype = GRL_F32;
    DeviceTensor(ContextPtr c, std::vector<py::ssize_t> s, int dt) : ctx(std::move(c)), shape(std::move(s)), dtype(dt) {
        buf = ctx->pool.acquire(std::max<size_t>(nbytes(), 16));
    }
    DeviceTensor(const DeviceTensor&) = delete;
    ~DeviceTensor() {
        if (buf.valid()) ctx->pool.release(buf);
    }
    size_t numel() const {
        size_t n = 1;
        for (auto d : shape) n *= size_t(d);
        return n;
    }
    size_t nbytes() const { return numel() * (dtype == GRL_BF16 ? 2 : 4); }
};
using TensorPtr = std::shared_ptr<DeviceTensor>;

static int parseDtype(const std::string& s) {
    if (s == "fp32" || s == "float32") return GRL_F32;
    if (s == "bf16" || s == "bfloat16") return GRL_BF16;
    throw std::runtime_error("dtype must be 'fp32' or 'bf16'");
}

static ops::RopeMode parseRopeMode(const std::string& m, bool allowNone) {
    if (m == "interleaved") return ops::RopeMode::Interleaved;
    if (m == "half" || m == "rotate_half") return ops::RopeMode::Half;
    if (allowNone && (m == "none" || m.empty())) return ops::RopeMode::None;
    throw std::runtime_error("rope_mode must be 'interleaved' or 'half'");
}

static py::array_t<float> flashImpl(GrillyCoreContext& ctx, FArr Q, FArr K, FArr V, std::optional<FArr> mask,
                                    float scale, bool causal, std::optional<IArr> seqLens, float ropeTheta,
                                    float ropeScaling, const std::string& ropeMode, const std::string& dtype,
                                    std::optional<py::array_t<float>> outArr = std::nullopt) {
    if (Q.ndim() != 4) throw std::runtime_error("Q must be 4D (batch, heads, seq_len, head_dim)");
    if (K.ndim() != 4 || V.ndim() != 4) throw std::runtime_error("K and V must be 4D (batch, heads, seq_len, head_dim)");
    for (int i = 0; i < 4; ++i)
        if (K.shape(i) != Q.shape(i) || V.shape(i) != Q.shape(i))
            throw std::runtime_error("Q, K and V must have the same shape");
    const uint32_t B = uint32_t(Q.shape(0)), H = uint32_t(Q.shape(1)), S = uint32_t(Q.shape(2)), D = uint32_t(Q.shape(3));
    ops::FlashAttention2Options opt;
    opt.causal = causal;
    const float* maskPtr = nullptr;
    if (mask.has_value()) {
        const auto& m = *mask;
        const bool ok2 = m.ndim() == 2 && m.shape(0) == B && m.shape(1) == S;
        const bool ok3 = m.ndim() == 3 && m.shape(0) == B && m.shape(1) == S && m.shape(2) == S;
        const bool ok4 = m.ndim() == 4 && m.shape(0) == B && (m.shape(1) == H || m.shape(1) == 1) && m.shape(2) == S &&
                         m.shape(3) == S;
        if (!ok2 && !ok3 && !ok4)
            throw std::runtime_error("mask must be (batch, seq), (batch, seq, seq) or (batch, heads|1, seq, seq)");
        opt.maskRank = int(m.ndim());
        opt.maskBroadcastHeads = ok4 && m.shape(1) == 1 && H != 1;
        maskPtr = m.data();
    }
    if (seqLens.has_value()) {
        if (seqLens->ndim() != 1 || seqLens->shape(0) != B) throw std::runtime_error("seq_lens must be (batch,)");
        opt.seqLens = seqLens->data();
    }
    if (ropeTheta != 0.0f) {
        opt.ropeMode = parseRopeMode(ropeMode, false);
        opt.ropeTheta = ropeTheta;
        opt.ropeScaling = ropeScaling;
    }
    if (dtype == "bf16") opt.precision = ops::Precision::BF16;
    else if (dtype != "fp32") throw std::runtime_error("dtype must be 'fp32' or 'bf16'");
    // out=: write into the caller's array (numpy style); a pinned host array there lets the download run
    // at the full PCIe rate and saves the first-touch page faults of a fresh 100+ MiB result
    py::array_t<float> result;
    if (outArr.has_value()) {
        result = *outArr;
        if (result.ndim() != 4 || result.shape(0) != B || result.shape(1) != H || result.shape(2) != S ||
            result.shape(3) != D || !(result.flags() & py::array::c_style) || !result.writeable())
            throw std::runtime_error("out must be a writable C-contiguous float32 array of Q's shape");
    } else {
        result = py::array_t<float>({py::ssize_t(B), py::ssize_t(H), py::ssize_t(S), py::ssize_t(D)});
    }
    float* out = result.mutable_data();
    const float *q = Q.data(), *k = K.data(), *v = V.data();
    {
        py::gil_scoped_release nogil;
        ops::flashAttention2Ex(ctx.batch, ctx.pool, ctx.cache, q, k, v, maskPtr, out, B, S, H, D, scale, opt);
    }
    return result;
}

PYBIND11_MODULE(grilly_core, m) {
    m.doc() = "grilly C++ backend, CUDA (sm_100a) build of the attention / KV-cache ops";
    m.attr("BACKEND") = "cuda-sm100a";

    py::class_<GrillyCoreContext, ContextPtr>(m, "Device")
        .def(py::init<>(), "Initialize the CUDA device, buffer pool and kernel-plan cache")
        .def(py::init<int>(), py::arg("gpu_index"), "Open the GPU with this ordinal")
        .def("synchronize",
             [](GrillyCoreContext& c) {
                 py::gil_scoped_release nogil;
                 check(grl_sync(c.device.handle(), 0), "Device.synchronize");
             },
             "Wait for the work queued on this device (DeviceTensor ops are asynchronous)")
        .def_property_readonly("gpu_index", [](const GrillyCoreContext& c) { return c.device.ordinal(); })
        .def("load_shaders", &GrillyCoreContext::loadShaders, py::arg("shader_dir"),
             "Accepted for compatibility; kernels are linked into the library")
        .def_property_readonly("device_name", [](const GrillyCoreContext& c) { return c.device.deviceName(); })
        .def_property_readonly("has_cooperative_matrix",
                               [](const GrillyCoreContext& c) { return c.device.hasCooperativeMatrix(); })
        .def_property_readonly("has_float16", [](const GrillyCoreContext& c) { return c.device.hasFloat16(); })
        .def_property_readonly("sm_count", [](const GrillyCoreContext& c) { return c.device.smCount(); })
        .def("pool_stats",
             [](const GrillyCoreContext& c) {
                 auto s = c.pool.stats();
                 py::dict d;
                 d["hits"] = s.hits; d["misses"] = s.misses; d["allocations"] = s.allocations;
                 d["total_acquired"] = s.totalAcquired; d["total_released"] = s.totalReleased;
                 return d;
             })
        .def("cache_stats", [](const GrillyCoreContext& c) {
            auto s = c.cache.cacheStats();
            py::dict d;
            d["hits"] = s.hits; d["misses"] = s.misses; d["evictions"] = s.evictions; d["cached_sets"] = s.cachedSets;
            return d;
        })
        // additive: the TMA descriptors the CUDA library keeps per (pointer, shape, box)
        .def("tensor_map_stats", [](const GrillyCoreContext& c) {
            auto s = c.cache.cacheStats();
            py::dict d;
            d["hits"] = s.tensorMapHits; d["misses"] = s.tensorMapMisses; d["cached"] = s.tensorMapsCached;
            return d;
        });

    // host-side rounding used by the chunked upload path (needs no GPU; exposed for the tests)
    m.def(
        "_host_round_bf16",
        [](FArr a) {
            py::array_t<uint16_t> out{py::ssize_t(a.size())};
            convertF32ToBF16(a.data(), out.mutable_data(), size_t(a.size()));
            return out;
        },
        py::arg("array"), "float32 -> bf16 bit patterns (round to nearest even) on the host worker threads");

    // ---- device-resident tensors
    py::class_<DeviceTensor, TensorPtr>(m, "DeviceTensor")
        .def_static(
            "from_numpy",
            [](ContextPtr ctx, FArr a, const std::string& dtype) {
                const int dt = parseDtype(dtype);
                std::vector<py::ssize_t> shape(a.shape(), a.shape() + a.ndim());
                auto t = std::make_shared<DeviceTensor>(ctx, shape, dt);
                const size_t n = t->numel();
                grl_device* dev = ctx->device.handle();
                if (dt == GRL_F32) {
                    check(grl_memcpy_h2d(dev, t->buf.dptr, a.data(), n * 4), "DeviceTensor.from_numpy");
                    check(grl_sync(dev, 0), "DeviceTensor.from_numpy");     // the source array may go away
                } else {
                    GrillyBuffer tmp = ctx->pool.acquire(std::max<size_t>(n * 4, 16));
                    check(grl_memcpy_h2d(dev, tmp.dptr, a.data(), n * 4), "DeviceTensor.from_numpy");
                    check(grl_cast(dev, tmp.dptr, GRL_F32, t->buf.dptr, GRL_BF16, n), "DeviceTensor.from_numpy");
                    check(grl_sync(dev, 0), "DeviceTensor.from_numpy");
                    ctx->pool.release(tmp);
                }
                return t;
            },
            py::arg("device"), py::arg("array"), py::arg("dtype") = "fp32",
            "Upload a float32 array (rounded to bf16 on the device when dtype='bf16')")
        .def_static(
            "empty",
            [](ContextPtr ctx, std::vector<py::ssize_t> shape, const std::string& dtype) {
                return std::make_shared<DeviceTensor>(ctx, shape, parseDtype(dtype));
            },
            py::arg("device"), py::arg("shape"), py::arg("dtype") = "fp32")
        .def(
            "to_numpy",
            [](DeviceTensor& t, std::optional<py::array_t<float>> outArr) {
                py::array_t<float> out;
                if (outArr.has_value()) {
                    out = *outArr;
                    if (size_t(out.size()) != t.numel() || !(out.flags() & py::array::c_style) || !out.writeable())
                        throw std::runtime_error("out must be a writable C-contiguous float32 array of the tensor's size");
                } else {
                    out = py::array_t<float>(t.shape);
                }
                grl_device* dev = t.ctx->device.handle();
                const size_t n = t.numel();
                float* dst = out.mutable_data();
                py::gil_scoped_release nogil;
                if (t.dtype == GRL_F32) {
                    check(grl_memcpy_d2h(dev, dst, t.buf.dptr, n * 4), "DeviceTensor.to_numpy");
                    check(grl_sync(dev, 0), "DeviceTensor.to_numpy");
                } else {
                    GrillyBuffer tmp = t.ctx->pool.acquire(std::max<size_t>(n * 4, 16));
                    check(grl_cast(dev, t.buf.dptr, GRL_BF16, tmp.dptr, GRL_F32, n), "DeviceTensor.to_numpy");
                    check(grl_memcpy_d2h(dev, dst, tmp.dptr, n * 4), "DeviceTensor.to_numpy");
                    check(grl_sync(dev, 0), "DeviceTensor.to_numpy");
                    t.ctx->pool.release(tmp);
                }
                return out;
            },
            py::arg("out") = py::none(), "Download as float32 (waits for the device)")
        .def(
            "copy_from_numpy",
            [](DeviceTensor& t, FArr a) {
                if (size_t(a.size()) != t.numel()) throw std::runtime_error("array size differs from the tensor's");
                if (t.dtype != GRL_F32) throw std::runtime_error("copy_from_numpy needs a float32 tensor");
                check(grl_memcpy_h2d(t.ctx->device.handle(), t.buf.dptr, a.data(), t.numel() * 4), "copy_from_numpy");
                check(grl_sync(t.ctx->device.handle(), 0), "copy_from_numpy");
            },
            py::arg("array"))
        .def_property_readonly("shape", [](const DeviceTensor& t) { return py::tuple(py::cast(t.shape)); })
        .def_property_readonly("dtype", [](const DeviceTensor& t) { return t.dtype == GRL_BF16 ? "bf16" : "fp32"; })
        .def_property_readonly("nbytes", [](const DeviceTensor& t) { return t.nbytes(); })
        .def_property_readonly("data_ptr", [](const DeviceTensor& t) { return reinterpret_cast<uintptr_t>(t.buf.dptr); })
        .def_property_readonly("device", [](const DeviceTensor& t) { return t.ctx; });

    // flash_attention2 on DeviceTensors: same keywords; Q/K/V (B,H,S,D) of one dtype (bf16 selects the
    // tcgen05 kernel), result a float32 DeviceTensor unless out= names one.  Asynchronous.
    m.def(
        "flash_attention2",
        [](ContextPtr ctx, TensorPtr Q, TensorPtr K, TensorPtr V, py::object mask, float scale, uint32_t, uint32_t,
           bool causal, std::optional<IArr> seqLens, float ropeTheta, float ropeScaling, const std::string& ropeMode,
           const std::string& /*dtype: taken from the tensors*/, std::optional<TensorPtr> out) {
            if (!mask.is_none()) throw std::runtime_error("DeviceTensor inputs take causal / seq_lens masks only");
            if (Q->shape.size() != 4) throw std::runtime_error("Q must be 4D (batch, heads, seq_len, head_dim)");
            if (K->shape != Q->shape || V->shape != Q->shape) throw std::runtime_error("Q, K and V must have the same shape");
            if (K->dtype != Q->dtype || V->dtype != Q->dtype) throw std::runtime_error("Q, K and V must have the same dtype");
            for (auto& t : {Q, K, V})
                if (t->ctx.get() != ctx.get()) throw std::runtime_error("tensor lives on another Device");
            const uint32_t B = uint32_t(Q->shape[0]), H = uint32_t(Q->shape[1]), S = uint32_t(Q->shape[2]),
                           D = uint32_t(Q->shape[3]);
            TensorPtr o = out.has_value() ? *out : std::make_shared<DeviceTensor>(ctx, Q->shape, GRL_F32);
            if (o->shape != Q->shape || o->ctx.get() != ctx.get()) throw std::runtime_error("out must have Q's shape and Device");
            GrillyBuffer lens;
            if (seqLens.has_value()) {
                if (seqLens->ndim() != 1 || seqLens->shape(0) != B) throw std::runtime_error("seq_lens must be (batch,)");
                lens = ctx->pool.acquire(size_t(B) * 4);
                ctx->pool.upload(lens, seqLens->data(), size_t(B) * 4);
                check(grl_sync(ctx->device.handle(), 0), "flash_attention2: seq_lens upload");
            }
            const ops::RopeMode mode = ropeTheta != 0.0f ? parseRopeMode(ropeMode, false) : ops::RopeMode::None;
            try {
                ops::flashAttention2Device(ctx->batch, ctx->cache, Q->buf, K->buf, V->buf, o->buf, Q->dtype, o->dtype, B, S,
                                           H, D, scale, causal, lens.valid() ? &lens : nullptr, mode,
                                           ropeTheta != 0.0f ? ropeTheta : 10000.0f, ropeScaling);
            } catch (...) {
                ctx->pool.release(lens);
                throw;
            }
            // stream order protects a pooled buffer that is handed out again; the pool waits before it frees one
            ctx->pool.release(lens);
            return o;
        },
        py::arg("device"), py::arg("Q"), py::arg("K"), py::arg("V"), py::arg("mask") = py::none(),
        py::arg("scale") = 0.0f, py::arg("tile_size_q") = 64, py::arg("tile_size_k") = 64, py::arg("causal") = false,
        py::arg("seq_lens") = py::none(), py::arg("rope_theta") = 0.0f, py::arg("rope_scaling") = 1.0f,
        py::arg("rope_mode") = "interleaved", py::arg("dtype") = "", py::arg("out") = py::none(),
        "Flash Attention 2 on DeviceTensors (asynchronous, result stays in HBM)");

    // ---- flash attention 2 (reference: bindings.cpp:416-462)
    m.def(
        "flash_attention2",
        [](GrillyCoreContext& ctx, FArr Q, FArr K, FArr V, std::optional<FArr> mask, float scale, uint32_t, uint32_t,
           bool causal, std::optional<IArr> seqLens, float ropeTheta, float ropeScaling, const std::string& ropeMode,
           const std::string& dtype, std::optional<py::array_t<float>> out) {
            return flashImpl(ctx, Q, K, V, mask, scale, causal, seqLens, ropeTheta, ropeScaling, ropeMode, dtype, out);
        },
        py::arg("device"), py::arg("Q"), py::arg("K"), py::arg("V"), py::arg("mask") = py::none(),
        py::arg("scale") = 0.0f, py::arg("tile_size_q") = 64, py::arg("tile_size_k") = 64, py::arg("causal") = false,
        py::arg("seq_lens") = py::none(), py::arg("rope_theta") = 0.0f, py::arg("rope_scaling") = 1.0f,
        py::arg("rope_mode") = "interleaved", py::arg("dtype") = "fp32", py::arg("out") = py::none(),
        "GPU Flash Attention 2 with online softmax tiling");

    m.def("set_pipeline_timing", &ops::setPipelineTiming, py::arg("on"),
          "Collect per-stage queue times in the chunked flash_attention2 host path (see last_pipeline_info)");
    m.def("last_pipeline_info", []() -> py::object {
        const auto i = ops::lastPipelineInfo();
        if (!i.valid) return py::none();
        py::dict d;
        d["host_cast_pct"] = i.hostCastPct; d["chunks"] = i.chunks; d["host_threads"] = i.hostThreads;
        d["host_round_ms"] = i.hostRoundMs; d["h2d_busy_ms"] = i.h2dMs; d["total_ms"] = i.totalMs;
        d["h2d_bytes"] = i.h2dBytes; d["d2h_bytes"] = i.d2hBytes;
        d["host_round_gbs"] = i.hostRoundMs > 0 ? i.hostRoundBytes / i.hostRoundMs * 1e-6 : 0.0;
        d["h2d_gbs"] = i.h2dMs > 0 ? i.h2dBytes / i.h2dMs * 1e-6 : 0.0;
        if (i.timed) {
            d["kernel_busy_ms"] = i.kernelMs; d["d2h_busy_ms"] = i.d2hMs;
            d["d2h_gbs"] = i.d2hMs > 0 ? i.d2hBytes / i.d2hMs * 1e-6 : 0.0;
        }
        return d;
    }, "Stages of this process's last chunked flash_attention2 call: share rounded on the host, busy time per stage");

    // ---- flash attention 2 + RoPE (push block of shaders/flash-attention2-rope.glsl:56-71)
    m.def(
        "flash_attention2_rope",
        [](GrillyCoreContext& ctx, FArr Q, FArr K, FArr V, std::optional<FArr> mask, float scale, float ropeBase,
           float ropeScaling, bool useRope, bool causal, std::optional<IArr> seqLens, const std::string& dtype) {
            return flashImpl(ctx, Q, K, V, mask, scale, causal, seqLens, useRope ? ropeBase : 0.0f, ropeScaling,
                             "interleaved", dtype);
        },
        py::arg("device"), py::arg("Q"), py::arg("K"), py::arg("V"), py::arg("mask") = py::none(),
        py::arg("scale") = 0.0f, py::arg("rope_base") = 10000.0f, py::arg("rope_scaling") = 1.0f,
        py::arg("use_rope") = true, py::arg("causal") = false, py::arg("seq_lens") = py::none(),
        py::arg("dtype") = "fp32", "Flash Attention 2 with interleaved-pair RoPE applied to Q and K");

    m.def(
        "rope",
        [](GrillyCoreContext& ctx, FArr x, float base, float scaling, std::optional<FArr> cosT,
           std::optional<FArr> sinT, const std::string& mode) {
            if (x.ndim() != 4) throw std::runtime_error("x must be 4D (batch, seq_len, heads, head_dim)");
            const uint32_t B = uint32_t(x.shape(0)), S = uint32_t(x.shape(1)), H = uint32_t(x.shape(2)),
                           D = uint32_t(x.shape(3));
            if (cosT.has_value() != sinT.has_value()) throw std::runtime_error("cos and sin tables go together");
            if (cosT.has_value() &&
                (cosT->ndim() != 2 || cosT->shape(0) < S || cosT->shape(1) != D / 2 || sinT->ndim() != 2 ||
                 sinT->shape(0) < S || sinT->shape(1) != D / 2))
                throw std::runtime_error("cos/sin tables must be (>= seq_len, head_dim/2)");
            py::array_t<float> y({py::ssize_t(B), py::ssize_t(S), py::ssize_t(H), py::ssize_t(D)});
            ops::rope(ctx.batch, ctx.pool, ctx.cache, x.data(), y.mutable_data(), B, S, H, D, base, scaling,
                      parseRopeMode(mode, false), cosT ? cosT->data() : nullptr, sinT ? sinT->data() : nullptr);
            return y;
        },
        py::arg("device"), py::arg("x"), py::arg("base") = 10000.0f, py::arg("scaling") = 1.0f,
        py::arg("cos") = py::none(), py::arg("sin") = py::none(), py::arg("mode") = "half",
        "RoPE on (batch, seq_len, heads, head_dim)");

    m.def(
        "attention_mask",
        [](GrillyCoreContext& ctx, FArr scores, std::optional<FArr> mask, bool causal, float maskValue) {
            if (scores.ndim() != 4 || scores.shape(2) != scores.shape(3))
                throw std::runtime_error("scores must be 4D (batch, heads, seq_len, seq_len)");
            const uint32_t B = uint32_t(scores.shape(0)), H = uint32_t(scores.shape(1)), S = uint32_t(scores.shape(2));
            if (!causal && !mask.has_value()) throw std::runtime_error("a (batch, seq_len) mask is required unless causal");
            if (mask.has_value() && (mask->ndim() != 2 || mask->shape(0) != B || mask->shape(1) != S))
                throw std::runtime_error("mask must be (batch, seq_len)");
            py::array_t<float> out({py::ssize_t(B), py::ssize_t(H), py::ssize_t(S), py::ssize_t(S)});
            std::memcpy(out.mutable_data(), scores.data(), size_t(B) * H * S * S * 4);
            ops::attentionMask(ctx.batch, ctx.pool, ctx.cache, out.mutable_data(), mask ? mask->data() : nullptr, B, H,
                               S, causal, maskValue);
            return out;
        },
        py::arg("device"), py::arg("scores"), py::arg("mask") = py::none(), py::arg("causal") = false,
        py::arg("mask_value") = -1e9f, "Causal or key-padding fill on attention scores; returns the masked copy");

    // ---- swizzle_kv (reference: bindings.cpp:784-832)
    m.def(
        "swizzle_kv",
        [](GrillyCoreContext& ctx, FArr input, uint32_t waveSize, bool reverse) -> py::array_t<float> {
            if (input.ndim() != 4) throw std::runtime_error("input must be 4D (batch, heads, seq_len, head_dim)");
            if (waveSize == 0) throw std::runtime_error("wave_size must be positive");
            const uint32_t B = uint32_t(input.shape(0)), H = uint32_t(input.shape(1)), S = uint32_t(input.shape(2)),
                           D = uint32_t(input.shape(3));
            py::array_t<float> result;
            if (reverse) {
                // the 4-D array holds swizzled data, which only has that many elements when nothing was padded
                if (S % waveSize || D % waveSize)
                    throw std::runtime_error("reverse needs seq_len and head_dim to be multiples of wave_size");
                result = py::array_t<float>({py::ssize_t(B), py::ssize_t(H), py::ssize_t(S), py::ssize_t(D)});
            } else {
                result = py::array_t<float>(py::ssize_t(ops::swizzledBufferSize(B, H, S, D, waveSize) / sizeof(float)));
            }
            ops::swizzle(ctx.batch, ctx.pool, ctx.cache, input.data(), result.mutable_data(), B, H, S, D, waveSize, reverse);
            return result;
        },
        py::arg("device"), py::arg("input"), py::arg("wave_size") = 32, py::arg("reverse") = false,
        "Swizzle/unswizzle KV tensor: [B,H,S,D] -> [B,H,S/W,D/W,W,W] (flat, zero padded) and back");

    // ---- the unfused attention pieces and the attention backward pass.  The reference dispatches these as shaders
    // from its Python backend (attention-scores, activation-softmax, attention-output(-gpt), attention-backward) and
    // has no pybind entry for them; the names follow VulkanBackwardOps.attention_backward
    // (src/grilly_next/backend/autograd_core.py:617-655) and the shader names.
    m.def(
        "attention_scores",
        [](GrillyCoreContext& ctx, FArr q, FArr k, float scale) -> py::array_t<float> {
            if (q.ndim() != 4 || k.ndim() != 4) throw std::runtime_error("q and k must be 4D (batch, seq_len, heads, head_dim)");
            for (int i = 0; i < 4; ++i)
                if (q.shape(i) != k.shape(i)) throw std::runtime_error("q and k shapes differ");
            const uint32_t B = uint32_t(q.shape(0)), S = uint32_t(q.shape(1)), H = uint32_t(q.shape(2)), D = uint32_t(q.shape(3));
            py::array_t<float> out({py::ssize_t(B), py::ssize_t(H), py::ssize_t(S), py::ssize_t(S)});
            ops::attentionScores(ctx.batch, ctx.pool, ctx.cache, q.data(), k.data(), out.mutable_data(), B, S, H, D, scale);
            return out;
        },
        py::arg("device"), py::arg("q"), py::arg("k"), py::arg("scale") = 0.0f,
        "scores (B,H,S,S) = scale * Q K^T for Q, K laid out (B,S,H,D); scale 0 means 1/sqrt(head_dim)");
    m.def(
        "softmax",
        [](GrillyCoreContext& ctx, FArr x) -> py::array_t<float> {
            if (x.ndim() < 1 || x.size() == 0) throw std::runtime_error("softmax: empty input");
            const uint32_t F = uint32_t(x.shape(x.ndim() - 1));
            std::vector<py::ssize_t> shape(x.shape(), x.shape() + x.ndim());
            py::array_t<float> out(shape);
            ops::softmax(ctx.batch, ctx.pool, ctx.cache, x.data(), out.mutable_data(), size_t(x.size()) / F, F);
            return out;
        },
        py::arg("device"), py::arg("x"), "Softmax over the last axis");
    m.def(
        "attention_output",
        [](GrillyCoreContext& ctx, FArr weights, FArr v, bool causal) -> py::array_t<float> {
            if (weights.ndim() != 4 || v.ndim() != 4)
                throw std::runtime_error("weights must be (batch, heads, seq_len, seq_len) and v (batch, seq_len, heads, head_dim)");
            const uint32_t B = uint32_t(v.shape(0)), S = uint32_t(v.shape(1)), H = uint32_t(v.shape(2)), D = uint32_t(v.shape(3));
            if (weights.shape(0) != B || weights.shape(1) != H || weights.shape(2) != S || weights.shape(3) != S)
                throw std::runtime_error("weights shape does not match v");
            py::array_t<float> out({py::ssize_t(B), py::ssize_t(S), py::ssize_t(H), py::ssize_t(D)});
            ops::attentionOutput(ctx.batch, ctx.pool, ctx.cache, weights.data(), v.data(), out.mutable_data(), B, S, H, D, causal);
            return out;
        },
        py::arg("device"), py::arg("weights"), py::arg("v"), py::arg("causal") = false,
        "out (B,S,H,D) = weights (B,H,S,S) . V (B,S,H,D); causal=True is the GPT form (sum over k <= q)");
    m.def(
        "attention_backward",
        [](GrillyCoreContext& ctx, FArr gradOutput, FArr q, FArr k, FArr v, FArr attn, float scale) -> py::tuple {
            if (q.ndim() != 4) throw std::runtime_error("q must be 4D (batch, heads, seq_len, head_dim)");
            const uint32_t B = uint32_t(q.shape(0)), H = uint32_t(q.shape(1)), S = uint32_t(q.shape(2)), D = uint32_t(q.shape(3));
            for (const FArr* t : {&gradOutput, &k, &v}) {
                if (t->ndim() != 4) throw std::runtime_error("grad_output, k and v must be 4D like q");
                for (int i = 0; i < 4; ++i)
                    if (t->shape(i) != q.shape(i)) throw std::runtime_error("grad_output, k and v must have the shape of q");
            }
            if (attn.ndim() != 4 || attn.shape(0) != B || attn.shape(1) != H || attn.shape(2) != S || attn.shape(3) != S)
                throw std::runtime_error("attn_weights must be (batch, heads, seq_len, seq_len)");
            std::vector<py::ssize_t> shape{py::ssize_t(B), py::ssize_t(H), py::ssize_t(S), py::ssize_t(D)};
            py::array_t<float> gq(shape), gk(shape), gv(shape);
            ops::attentionBackward(ctx.batch, ctx.pool, ctx.cache, gradOutput.data(), q.data(), k.data(), v.data(), attn.data(),
                                   gq.mutable_data(), gk.mutable_data(), gv.mutable_data(), B, H, S, D, scale);
            return py::make_tuple(gq, gk, gv);
        },
        py::arg("device"), py::arg("grad_output"), py::arg("q"), py::arg("k"), py::arg("v"), py::arg("attn_weights"),
        py::arg("scale") = 0.0f, "(grad_q, grad_k, grad_v) of softmax(scale Q K^T) V; all tensors (B,H,S,D)");

    // ---- KV cache (reference: bindings.cpp:592-694)
    py::class_<ops::KVCache>(m, "KVCache")
        .def_readonly("current_len", &ops::KVCache::currentLen)
        .def_property_readonly("seq_lens", [](const ops::KVCache& kv) { return kv.hostSeqLens; })
        .def("stats", [](const ops::KVCache& kv) {
            auto s = ops::kvCacheGetStats(kv);
            py::dict d;
            d["current_tokens"] = s.currentTokens; d["max_tokens"] = s.maxTokens;
            d["total_evicted"] = s.totalEvicted; d["total_appended"] = s.totalAppended;
            d["compression_ratio"] = s.compressionRatio; d["avg_attention_score"] = s.avgAttentionScore;
            d["pages_total"] = s.pagesTotal; d["pages_used"] = s.pagesUsed; d["bytes"] = s.bytes;
            return d;
        });

    m.def(
        "create_kv_cache",
        [](GrillyCoreContext& ctx, uint32_t maxSeqLen, uint32_t numHeads, uint32_t headDim, uint32_t numLayers,
           uint32_t compressionRatio, uint32_t maxCacheTokens, bool useAsymmetricQuant, uint32_t valueBits,
           bool crossLayerSharing, bool useH2O, bool useSpeculativeEviction, float evictionThreshold,
           uint32_t batchSize, uint32_t pageTokens, const std::string& dtype) {
            ops::KVCacheConfig cfg;
            cfg.maxSeqLen = maxSeqLen; cfg.numHeads = numHeads; cfg.headDim = headDim; cfg.numLayers = numLayers;
            cfg.compressionRatio = compressionRatio; cfg.maxCacheTokens = maxCacheTokens;
            cfg.useAsymmetricQuant = useAsymmetricQuant; cfg.valueBits = valueBits;
            cfg.crossLayerSharing = crossLayerSharing; cfg.useH2O = useH2O;
            cfg.useSpeculativeEviction = useSpeculativeEviction; cfg.evictionThreshold = evictionThreshold;
            cfg.batchSize = batchSize; cfg.pageTokens = pageTokens;
            if (dtype == "bf16") cfg.dtype = GRL_BF16;
            else if (dtype == "fp32") cfg.dtype = GRL_F32;
            else throw std::runtime_error("dtype must be 'bf16' or 'fp32'");
            return ops::createKVCache(ctx.pool, cfg);
        },
        py::arg("device"), py::arg("max_seq_len") = 2048, py::arg("num_heads") = 8, py::arg("head_dim") = 64,
        py::arg("num_layers") = 12, py::arg("compression_ratio") = 4, py::arg("max_cache_tokens") = 2048,
        py::arg("use_asymmetric_quant") = false, py::arg("value_bits") = 4, py::arg("cross_layer_sharing") = false,
        py::arg("use_h2o") = true, py::arg("use_speculative_eviction") = false, py::arg("eviction_threshold") = 0.1f,
        py::arg("batch_size") = 1, py::arg("page_tokens") = 64, py::arg("dtype") = "bf16",
        "Create a KV cache (compression_ratio=1 selects the paged head-major cache built here; with "
        "use_asymmetric_quant=True its pages hold FP8-E4M3 keys, INT4 values and float16 group scales)");

    m.def("destroy_kv_cache",
          [](GrillyCoreContext& ctx, ops::KVCache& kv) { ops::destroyKVCache(ctx.pool, kv); }, py::arg("device"),
          py::arg("kv_cache"));

    auto checkNew = [](const ops::KVCache& kv, const FArr& a, const char* name, uint32_t heads) -> uint32_t {
        const auto& c = kv.config;
        if (a.ndim() == 3) {
            if (c.batchSize != 1) throw std::runtime_error(std::string(name) + " must be (batch, n, heads, head_dim) for a batched cache");
            if (a.shape(1) != heads || a.shape(2) != c.headDim)
                throw std::runtime_error(std::string(name) + " must be (n, heads, head_dim)");
            return uint32_t(a.shape(0));
        }
        if (a.ndim() == 4) {
            if (a.shape(0) != c.batchSize || a.shape(2) != heads || a.shape(3) != c.headDim)
                throw std::runtime_error(std::string(name) + " must be (batch, n, heads, head_dim)");
            return uint32_t(a.shape(1));
        }
        throw std::runtime_error(std::string(name) + " must be 3D or 4D");
    };

    m.def(
        "kv_cache_append",
        [checkNew](GrillyCoreContext& ctx, ops::KVCache& kv, FArr newKeys, FArr newValues, float ropeTheta,
                   float ropeScaling, const std::string& ropeMode) {
            const uint32_t n = checkNew(kv, newKeys, "new_keys", kv.config.numHeads);
            if (checkNew(kv, newValues, "new_values", kv.config.numHeads) != n)
                throw std::runtime_error("new_keys and new_values differ in length");
            if (ropeTheta != 0.0f)
                ops::kvCacheAppendRope(ctx.batch, ctx.pool, ctx.cache, kv, newKeys.data(), newValues.data(), n, nullptr,
                                       nullptr, 0, parseRopeMode(ropeMode, false), ropeTheta, ropeScaling);
            else
                ops::kvCacheAppend(ctx.batch, ctx.pool, ctx.cache, kv, newKeys.data(), newValues.data(), n);
        },
        py::arg("device"), py::arg("kv_cache"), py::arg("new_keys"), py::arg("new_values"),
        py::arg("rope_theta") = 0.0f, py::arg("rope_scaling") = 1.0f, py::arg("rope_mode") = "interleaved",
        "Append new KV pairs to the cache");

    m.def(
        "kv_cache_decode",
        [](GrillyCoreContext& ctx, const ops::KVCache& kv, uint32_t seq) {
            const auto& c = kv.config;
            if (seq >= c.batchSize) throw std::runtime_error("seq out of range");
            const py::ssize_t T = kv.hostSeqLens.empty() ? 0 : kv.hostSeqLens[seq];
            py::array_t<float> keys({T, py::ssize_t(c.numHeads), py::ssize_t(c.headDim)});
            py::array_t<float> values({T, py::ssize_t(c.numHeads), py::ssize_t(c.headDim)});
            ops::kvCacheDecode(ctx.batch, ctx.pool, ctx.cache, kv, keys.mutable_data(), values.mutable_data(), seq);
            py::dict r;
            r["keys"] = keys;
            r["values"] = values;
            return r;
        },
        py::arg("device"), py::arg("kv_cache"), py::arg("seq") = 0, "Decode KV from the cache as (T, heads, head_dim)");

    m.def(
        "kv_cache_evict_h2o",
        [](GrillyCoreContext& ctx, ops::KVCache& kv, std::optional<FArr> scores, uint32_t numEvict) {
            if (scores.has_value()) {
                const py::ssize_t T = kv.hostSeqLens.empty() ? 0 : kv.hostSeqLens[0];
                const bool ok2 = scores->ndim() == 2 && kv.config.batchSize == 1 && scores->shape(0) == T && scores->shape(1) == T;
                const bool ok3 = scores->ndim() == 3 && scores->shape(0) == kv.config.batchSize && scores->shape(1) == T &&
                                 scores->shape(2) == T;
                if (!ok2 && !ok3)
                    throw std::runtime_error("attention_scores must be (cache_len, cache_len), or (batch, cache_len, cache_len)");
            }
            ops::kvCacheEvictH2O(ctx.batch, ctx.pool, ctx.cache, kv, scores ? scores->data() : nullptr, numEvict);
        },
        py::arg("device"), py::arg("kv_cache"), py::arg("attention_scores") = py::none(), py::arg("num_evict") = 0,
        "Add the column sums of attention_scores to the cumulative scores, tombstone the num_evict lowest");
    m.def("kv_cache_compact",
          [](GrillyCoreContext& ctx, ops::KVCache& kv) { ops::kvCacheCompact(ctx.batch, ctx.pool, ctx.cache, kv); },
          py::arg("device"), py::arg("kv_cache"), "Move the live tokens to the front and shrink the cache length");
    m.def(
        "kv_cache_init_eviction_head",
        [](GrillyCoreContext& ctx, ops::KVCache& kv, uint32_t inputDim, uint32_t hiddenDim, float lr) {
            ops::kvCacheInitEvictionHead(ctx.pool, kv, inputDim, hiddenDim, lr);
        },
        py::arg("device"), py::arg("kv_cache"), py::arg("input_dim"), py::arg("hidden_dim") = 32, py::arg("lr") = 1e-3f,
        "Initialize trainable eviction head for speculative eviction");
    m.def(
        "kv_cache_train_eviction_head",
        [](GrillyCoreContext& ctx, ops::KVCache& kv, FArr tokenFeatures, FArr attentionScores, uint32_t seqLen) {
            const auto& head = kv.evictionHead;
            if (head.initialized) {
                if (size_t(tokenFeatures.size()) != size_t(kv.currentLen) * head.inputDim)
                    throw std::runtime_error("token_features must be (cache_len, input_dim)");
                if (size_t(attentionScores.size()) != size_t(seqLen) * kv.currentLen)
                    throw std::runtime_error("attention_scores must be (seq_len, cache_len)");
            }
            ops::kvCacheTrainEvictionHead(ctx.batch, ctx.pool, ctx.cache, kv, tokenFeatures.data(), attentionScores.data(),
                                          seqLen);
        },
        py::arg("device"), py::arg("kv_cache"), py::arg("token_features"), py::arg("attention_scores"), py::arg("seq_len"),
        "Train the eviction head on attention patterns from latest forward pass");
    m.def(
        "kv_cache_eviction_head_weights",
        [](GrillyCoreContext& ctx, ops::KVCache& kv, std::optional<py::dict> set) {
            auto& head = kv.evictionHead;
            if (!head.initialized) throw std::runtime_error("the eviction head is not initialized");
            grl_device* dev = ctx.device.handle();
            const size_t n1 = size_t(head.inputDim) * head.hiddenDim, nh = head.hiddenDim;
            if (set.has_value()) {
                auto put = [&](const char* key, GrillyBuffer& buf, size_t n) {
                    if (!set->contains(key)) return;
                    FArr a = (*set)[key].cast<FArr>();
                    if (size_t(a.size()) != n) throw std::runtime_error(std::string(key) + " has the wrong size");
                    check(grl_memcpy_h2d(dev, buf.dptr, a.data(), n * 4), "eviction head weights");
                    check(grl_sync(dev, 0), "eviction head weights");
                };
                put("w1", head.w1, n1); put("b1", head.b1, nh); put("w2", head.w2, nh); put("b2", head.b2, 1);
            }
            py::array_t<float> w1({py::ssize_t(head.inputDim), py::ssize_t(head.hiddenDim)});
            py::array_t<float> b1{py::ssize_t(nh)}, w2{py::ssize_t(nh)}, b2{py::ssize_t(1)};
            check(grl_memcpy_d2h(dev, w1.mutable_data(), head.w1.dptr, n1 * 4), "eviction head weights");
            check(grl_memcpy_d2h(dev, b1.mutable_data(), head.b1.dptr, nh * 4), "eviction head weights");
            check(grl_memcpy_d2h(dev, w2.mutable_data(), head.w2.dptr, nh * 4), "eviction head weights");
            check(grl_memcpy_d2h(dev, b2.mutable_data(), head.b2.dptr, 4), "eviction head weights");
            check(grl_sync(dev, 0), "eviction head weights");
            py::dict d;
            d["w1"] = w1; d["b1"] = b1; d["w2"] = w2; d["b2"] = b2; d["total_updates"] = head.totalUpdates;
            return d;
        },
        py::arg("device"), py::arg("kv_cache"), py::arg("set") = py::none(),
        "Read (and optionally overwrite) the eviction head's parameters");
    m.def(
        "kv_cache_evict_speculative",
        [](GrillyCoreContext& ctx, ops::KVCache& kv, std::optional<FArr> hiddenStates, uint32_t hiddenDim) {
            const auto& head = kv.evictionHead;
            if (hiddenStates.has_value() && head.initialized && head.totalUpdates > 0 &&
                size_t(hiddenStates->size()) != size_t(kv.currentLen) * head.inputDim)
                throw std::runtime_error("hidden_states must be (cache_len, input_dim of the eviction head)");
            ops::kvCacheEvictSpeculative(ctx.batch, ctx.pool, ctx.cache, kv,
                                         hiddenStates ? hiddenStates->data() : nullptr, hiddenDim);
        },
        py::arg("device"), py::arg("kv_cache"), py::arg("hidden_states") = py::none(), py::arg("hidden_dim") = 64,
        "Run speculative eviction using trained auxiliary head (heuristic relevance until it has been trained)");
    m.def(
        "kv_cache_token_meta",
        [](GrillyCoreContext& ctx, const ops::KVCache& kv, uint32_t seq) {
            std::vector<float> cum, rel;
            std::vector<uint8_t> tomb;
            ops::kvCacheTokenMeta(ctx.pool, kv, seq, cum, tomb, rel);
            py::dict d;
            d["cumulative_score"] = py::array_t<float>(py::ssize_t(cum.size()), cum.data());
            d["tombstone"] = py::array_t<uint8_t>(py::ssize_t(tomb.size()), tomb.data());
            d["predicted_relevance"] = py::array_t<float>(py::ssize_t(rel.size()), rel.data());
            return d;
        },
        py::arg("device"), py::arg("kv_cache"), py::arg("seq") = 0, "Per-token eviction metadata of one sequence");

    // ---- GQA decode on DeviceTensors (asynchronous; q already rotated)
    m.def(
        "gqa_attention",
        [](ContextPtr ctx, TensorPtr q, ops::KVCache& kv, py::object vCache, py::object cacheLen, float scale,
           int nSplits, const std::string&) {
            if (!vCache.is_none() || !cacheLen.is_none())
                throw std::runtime_error("a DeviceTensor q attends over a KVCache; v_cache / cache_len do not apply");
            if (q->dtype != GRL_F32 || q->shape.size() != 4 || q->shape[1] != 1)
                throw std::runtime_error("q must be a float32 DeviceTensor (batch, 1, num_q_heads, head_dim)");
            if (q->shape[0] != kv.config.batchSize || q->shape[3] != kv.config.headDim)
                throw std::runtime_error("q does not match the cache");
            auto out = std::make_shared<DeviceTensor>(ctx, q->shape, GRL_F32);
            GrillyBuffer ws;
            ops::gqaAttentionDevice(ctx->pool, ctx->cache, kv, q->buf, out->buf, uint32_t(q->shape[2]), scale, nSplits, ws);
            ctx->pool.release(ws);
            return out;
        },
        py::arg("device"), py::arg("q"), py::arg("k_cache"), py::arg("v_cache") = py::none(),
        py::arg("cache_len") = py::none(), py::arg("scale") = 0.0f, py::arg("n_splits") = 0, py::arg("dtype") = "fp32",
        "GQA decode attention of a DeviceTensor q over a KVCache (asynchronous)");

    m.def(
        "decode_step",
        [](ContextPtr ctx, ops::KVCache& kv, TensorPtr q, TensorPtr kNew, TensorPtr vNew, float ropeTheta,
           float ropeScaling, const std::string& ropeMode, float scale) {
            const auto& c = kv.config;
            for (auto& t : {q, kNew, vNew})
                if (t->dtype != GRL_F32 || t->shape.size() != 4 || t->shape[0] != c.batchSize || t->shape[1] != 1 ||
                    t->shape[3] != c.headDim)
                    throw std::runtime_error("q / k_new / v_new must be float32 DeviceTensors (batch, 1, heads, head_dim)");
            if (kNew->shape[2] != c.numHeads || vNew->shape[2] != c.numHeads)
                throw std::runtime_error("k_new / v_new must be (batch, 1, num_kv_heads, head_dim)");
            auto out = std::make_shared<DeviceTensor>(ctx, q->shape, GRL_F32);
            GrillyBuffer qRot = ctx->pool.acquire(q->nbytes()), ws;
            try {
                ops::decodeStepDevice(ctx->pool, ctx->cache, kv, q->buf, kNew->buf, vNew->buf, qRot, out->buf,
                                      uint32_t(q->shape[2]),
                                      ropeTheta != 0.0f ? parseRopeMode(ropeMode, false) : ops::RopeMode::None,
                                      ropeTheta != 0.0f ? ropeTheta : 10000.0f, ropeScaling, scale, ws);
            } catch (...) {
                ctx->pool.release(qRot);
                ctx->pool.release(ws);
                throw;
            }
            ctx->pool.release(qRot);
            ctx->pool.release(ws);
            return out;
        },
        py::arg("device"), py::arg("kv_cache"), py::arg("q"), py::arg("k_new"), py::arg("v_new"),
        py::arg("rope_theta") = 10000.0f, py::arg("rope_scaling") = 1.0f, py::arg("rope_mode") = "interleaved",
        py::arg("scale") = 0.0f, "One decode step on DeviceTensors (asynchronous)");

    // ---- GQA decode (shaders/gqa-attention.glsl)
    m.def(
        "gqa_attention",
        [](GrillyCoreContext& ctx, FArr q, py::object kvOrK, std::optional<FArr> vCache, std::optional<uint32_t> cacheLen,
           float scale, int nSplits, const std::string& dtype, bool accumulateScores) {
            if (q.ndim() != 4 || q.shape(1) != 1) throw std::runtime_error("q must be (batch, 1, num_q_heads, head_dim)");
            const uint32_t B = uint32_t(q.shape(0)), Hq = uint32_t(q.shape(2)), D = uint32_t(q.shape(3));
            py::array_t<float> out({py::ssize_t(B), py::ssize_t(1), py::ssize_t(Hq), py::ssize_t(D)});
            if (py::isinstance<ops::KVCache>(kvOrK)) {
                auto& kv = kvOrK.cast<ops::KVCache&>();
                if (kv.config.batchSize != B || kv.config.headDim != D) throw std::runtime_error("q does not match the cache");
                ops::gqaAttention(ctx.batch, ctx.pool, ctx.cache, kv, q.data(), out.mutable_data(), Hq, scale, nSplits,
                                  accumulateScores);
                return out;
            }
            if (accumulateScores) throw std::runtime_error("accumulate_scores needs a KVCache (explicit arrays have no metadata)");
            // explicit (B,T,Hkv,D) arrays in the reference shader's layout: stage them in a temporary cache
            FArr kC = kvOrK.cast<FArr>();
            if (!vCache.has_value()) throw std::runtime_error("v_cache is required with an explicit k_cache");
            if (kC.ndim() != 4 || vCache->ndim() != 4 || kC.shape(0) != B || kC.shape(3) != D)
                throw std::runtime_error("k_cache / v_cache must be (batch, cache_len, num_kv_heads, head_dim)");
            for (int i = 0; i < 4; ++i)
                if (kC.shape(i) != vCache->shape(i)) throw std::runtime_error("k_cache and v_cache differ in shape");
            const uint32_t Tmax = uint32_t(kC.shape(1)), Hkv = uint32_t(kC.shape(2));
            const uint32_t T = cacheLen.value_or(Tmax);
            if (T == 0 || T > Tmax) throw std::runtime_error("cache_len out of range");
            if (Hkv == 0 || Hq % Hkv != 0) throw std::runtime_error("num_q_heads must be a multiple of num_kv_heads");
            ops::KVCacheConfig cfg;
            cfg.numHeads = Hkv; cfg.headDim = D; cfg.batchSize = B; cfg.maxCacheTokens = T; cfg.maxSeqLen = T;
            cfg.dtype = dtype == "bf16" ? GRL_BF16 : GRL_F32;
            ops::KVCache kv = ops::createKVCache(ctx.pool, cfg);
            try {
                if (T == Tmax) {
                    ops::kvCacheAppend(ctx.batch, ctx.pool, ctx.cache, kv, kC.data(), vCache->data(), T);
                } else {  // keep only the first T tokens of every sequence
                    std::vector<float> kk(size_t(B) * T * Hkv * D), vv(kk.size());
                    const size_t row = size_t(Hkv) * D;
                    for (uint32_t b = 0; b < B; ++b) {
                        std::memcpy(&kk[size_t(b) * T * row], kC.data() + size_t(b) * Tmax * row, size_t(T) * row * 4);
                        std::memcpy(&vv[size_t(b) * T * row], vCache->data() + size_t(b) * Tmax * row, size_t(T) * row * 4);
                    }
                    ops::kvCacheAppend(ctx.batch, ctx.pool, ctx.cache, kv, kk.data(), vv.data(), T);
                }
                ops::gqaAttention(ctx.batch, ctx.pool, ctx.cache, kv, q.data(), out.mutable_data(), Hq, scale, nSplits);
            } catch (...) {
                ops::destroyKVCache(ctx.pool, kv);
                throw;
            }
            ops::destroyKVCache(ctx.pool, kv);
            return out;
        },
        py::arg("device"), py::arg("q"), py::arg("k_cache"), py::arg("v_cache") = py::none(),
        py::arg("cache_len") = py::none(), py::arg("scale") = 0.0f, py::arg("n_splits") = 0, py::arg("dtype") = "fp32",
        py::arg("accumulate_scores") = false,
        "GQA decode attention: q (B,1,Hq,D) over a KVCache, or over explicit (B,T,Hkv,D) arrays; "
        "accumulate_scores adds the attention mass each cached token received to its H2O score");

    m.def(
        "decode_step",
        [](GrillyCoreContext& ctx, ops::KVCache& kv, FArr q, FArr kNew, FArr vNew, float ropeTheta, float ropeScaling,
           const std::string& ropeMode, float scale, std::optional<py::array_t<float>> outArr, bool accumulateScores) {
            const auto& c = kv.config;
            if (q.ndim() != 4 || q.shape(0) != c.batchSize || q.shape(1) != 1 || q.shape(3) != c.headDim)
                throw std::runtime_error("q must be (batch, 1, num_q_heads, head_dim)");
            for (const FArr* a : {&kNew, &vNew})
                if (a->ndim() != 4 || a->shape(0) != c.batchSize || a->shape(1) != 1 || a->shape(2) != c.numHeads ||
                    a->shape(3) != c.headDim)
                    throw std::runtime_error("k_new / v_new must be (batch, 1, num_kv_heads, head_dim)");
            const uint32_t Hq = uint32_t(q.shape(2));
            py::array_t<float> out;
            if (outArr.has_value()) {   // numpy style: a caller-owned (pinned) array saves the allocation and its page faults
                out = *outArr;
                if (out.size() != q.size() || !(out.flags() & py::array::c_style) || !out.writeable())
                    throw std::runtime_error("out must be a writable C-contiguous float32 array of q's size");
            } else {
                out = py::array_t<float>({py::ssize_t(c.batchSize), py::ssize_t(1), py::ssize_t(Hq), py::ssize_t(c.headDim)});
            }
            ops::decodeStep(ctx.batch, ctx.pool, ctx.cache, kv, q.data(), kNew.data(), vNew.data(), out.mutable_data(),
                            Hq, ropeTheta != 0.0f ? parseRopeMode(ropeMode, false) : ops::RopeMode::None,
                            ropeTheta != 0.0f ? ropeTheta : 10000.0f, ropeScaling, scale, accumulateScores);
            return out;
        },
        py::arg("device"), py::arg("kv_cache"), py::arg("q"), py::arg("k_new"), py::arg("v_new"),
        py::arg("rope_theta") = 10000.0f, py::arg("rope_scaling") = 1.0f, py::arg("rope_mode") = "interleaved",
        py::arg("scale") = 0.0f, py::arg("out") = py::none(), py::arg("accumulate_scores") = false,
        "RoPE(q,k) at the current position, append k/v, attend over the cache");

    // ---- KV-sharded decode across processes (one per GPU): NCCL behind the C ABI
    struct PyShardGroup {
        ContextPtr ctx;
        ops::ShardGroup g;
        ~PyShardGroup() { ops::destroyShardGroup(ctx->pool, g); }
    };
    m.def("shard_group_unique_id", []() {
        auto id = ops::shardGroupUniqueId();
        return py::bytes(reinterpret_cast<const char*>(id.data()), id.size());
    }, "128-byte id that rank 0 creates and hands to the other ranks before ShardGroup(...)");
    m.def("shard_range", [](uint64_t total, int world, int rank) { return ops::shardRange(total, world, rank); },
          py::arg("total_tokens"), py::arg("world"), py::arg("rank"), "Contiguous [start, end) of a rank's tokens");
    py::class_<PyShardGroup, std::shared_ptr<PyShardGroup>>(m, "ShardGroup")
        .def(py::init([](ContextPtr ctx, py::bytes id, int rank, int world) {
                 const std::string raw = id;
                 if (raw.size() != 128) throw std::runtime_error("ShardGroup: the id must be the 128 bytes of shard_group_unique_id()");
                 auto g = std::make_shared<PyShardGroup>();
                 g->ctx = ctx;
                 {
                     py::gil_scoped_release nogil;
                     g->g = ops::createShardGroup(ctx->device, reinterpret_cast<const uint8_t*>(raw.data()), rank, world);
                 }
                 return g;
             }),
             py::arg("device"), py::arg("unique_id"), py::arg("rank"), py::arg("world"),
             "Collective: every rank constructs it with the same id")
        .def_property_readonly("rank", [](const PyShardGroup& g) { return g.g.rank; })
        .def_property_readonly("world", [](const PyShardGroup& g) { return g.g.world; });
    m.def(
        "sharded_decode_step",
        [](ContextPtr ctx, ops::KVCache& kv, std::shared_ptr<PyShardGroup> group, FArr q, float scale,
           std::optional<py::array_t<float>> outArr, double timeoutMs) {
            const auto& c = kv.config;
            if (q.ndim() != 4 || q.shape(0) != c.batchSize || q.shape(1) != 1 || q.shape(3) != c.headDim)
                throw std::runtime_error("q must be (batch, 1, num_q_heads, head_dim)");
            const uint32_t Hq = uint32_t(q.shape(2));
            py::array_t<float> out;
            if (outArr.has_value()) {
                out = *outArr;
                if (out.size() != q.size() || !(out.flags() & py::array::c_style) || !out.writeable())
                    throw std::runtime_error("out must be a writable C-contiguous float32 array of q's size");
            } else {
                out = py::array_t<float>({py::ssize_t(c.batchSize), py::ssize_t(1), py::ssize_t(Hq), py::ssize_t(c.headDim)});
            }
            const float* qp = q.data();
            float* op = out.mutable_data();
            {
                py::gil_scoped_release nogil;
                ops::shardedDecodeStep(ctx->batch, ctx->pool, ctx->cache, kv, group->g, qp, op, Hq, scale,
                                       uint64_t(timeoutMs * 1e6));
            }
            return out;
        },
        py::arg("device"), py::arg("kv_cache"), py::arg("group"), py::arg("q"), py::arg("scale") = 0.0f,
        py::arg("out") = py::none(), py::arg("timeout_ms") = 2000.0,
        "Decode step over a KV cache sharded across the group's GPUs: local decode, NCCL all-gather of the partials, merge");

    // ---- DeviceGroup: the GPUs of one node behind one object, one Device (own stream, own pool) each.
    // flash_attention2 splits the heads in contiguous runs over the devices, one host thread per device
    // (heads are independent: no collective); the KV-sharded decode across processes lives in
    // grilly_next.parallel.
    struct DeviceGroup {
        std::vector<ContextPtr> devices;
    };
    py::class_<DeviceGroup>(m, "DeviceGroup")
        .def(py::init([](int n) {
                 int have = 0;
                 check(grl_device_count(&have), "DeviceGroup");
                 if (n <= 0) n = have;
                 if (n > have) throw std::runtime_error("DeviceGroup: " + std::to_string(n) + " devices asked for, " +
                                                        std::to_string(have) + " present");
                 auto g = std::make_unique<DeviceGroup>();
                 for (int i = 0; i < n; ++i) g->devices.push_back(std::make_shared<GrillyCoreContext>(i));
                 return g;
             }),
             py::arg("n") = 0, "Open the first n GPUs (0 = all)")
        .def("__len__", [](const DeviceGroup& g) { return g.devices.size(); })
        .def("__getitem__",
             [](const DeviceGroup& g, size_t i) {
                 if (i >= g.devices.size()) throw py::index_error();
                 return g.devices[i];
             })
        .def_property_readonly("devices", [](const DeviceGroup& g) { return g.devices; })
        .def(
            "flash_attention2",
            [](DeviceGroup& g, FArr Q, FArr K, FArr V, float scale, bool causal, std::optional<IArr> seqLens,
               float ropeTheta, float ropeScaling, const std::string& ropeMode, const std::string& dtype) {
                if (Q.ndim() != 4) throw std::runtime_error("Q must be 4D (batch, heads, seq_len, head_dim)");
                for (int i = 0; i < 4; ++i)
                    if (K.ndim() != 4 || V.ndim() != 4 || K.shape(i) != Q.shape(i) || V.shape(i) != Q.shape(i))
                        throw std::runtime_error("Q, K and V must have the same shape");
                const uint32_t B = uint32_t(Q.shape(0)), H = uint32_t(Q.shape(1)), S = uint32_t(Q.shape(2)),
                               D = uint32_t(Q.shape(3));
                if (seqLens.has_value() && (seqLens->ndim() != 1 || seqLens->shape(0) != B))
                    throw std::runtime_error("seq_lens must be (batch,)");
                ops::FlashAttention2Options opt;
                opt.causal = causal;
                if (seqLens.has_value()) opt.seqLens = seqLens->data();
                if (ropeTheta != 0.0f) {
                    opt.ropeMode = parseRopeMode(ropeMode, false);
                    opt.ropeTheta = ropeTheta;
                    opt.ropeScaling = ropeScaling;
                }
                opt.precision = parseDtype(dtype) == GRL_BF16 ? ops::Precision::BF16 : ops::Precision::FP32;
                py::array_t<float> result({py::ssize_t(B), py::ssize_t(H), py::ssize_t(S), py::ssize_t(D)});
                float* out = result.mutable_data();
                const float *q = Q.data(), *k = K.data(), *v = V.data();
                const size_t G = g.devices.size(), slice = size_t(S) * D;
                std::vector<std::string> errors(G);
                {
                    py::gil_scoped_release nogil;
                    std::vector<std::thread> workers;
                    for (size_t r = 0; r < G; ++r) {
                        const uint32_t h0 = uint32_t(size_t(H) * r / G), h1 = uint32_t(size_t(H) * (r + 1) / G);
                        if (h1 == h0) continue;
                        workers.emplace_back([&, r, h0, h1] {
                            try {
                                auto& c = *g.devices[r];
                                // every (batch) row of this device's head run is one call: (1, h1-h0, S, D) is contiguous
                                for (uint32_t b = 0; b < B; ++b) {
                                    const size_t off = (size_t(b) * H + h0) * slice;
                                    ops::FlashAttention2Options o = opt;
                                    if (opt.seqLens) o.seqLens = opt.seqLens + b;
                                    ops::flashAttention2Ex(c.batch, c.pool, c.cache, q + off, k + off, v + off, nullptr,
                                                           out + off, 1, S, h1 - h0, D, scale, o);
                                }
                            } catch (const std::exception& e) {
                                errors[r] = e.what();
                            }
                        });
                    }
                    for (auto& w : workers) w.join();
                }
                for (auto& e : errors)
                    if (!e.empty()) throw std::runtime_error(e);
                return result;
            },
            py::arg("Q"), py::arg("K"), py::arg("V"), py::arg("scale") = 0.0f, py::arg("causal") = false,
            py::arg("seq_lens") = py::none(), py::arg("rope_theta") = 0.0f, py::arg("rope_scaling") = 1.0f,
            py::arg("rope_mode") = "interleaved", py::arg("dtype") = "fp32",
            "Flash Attention 2 with the heads split over the group's GPUs");

    // ---- names of the reference's module that this build does not implement: present, and say so
    auto notBuilt = [&m](const char* name, const char* what) {
        const std::string msg = std::string(name) + ": " + what;
        m.def(name, [msg](py::args, py::kwargs) -> py::object { throw std::runtime_error(msg); });
    };
    // ---- CPU reference of the MLA path (cpp/python/bindings.cpp:838-899 there): same signature, same shape rules
    m.def(
        "fused_attention_cpu",
        [](FArr Q, FArr latents, FArr wUp, std::optional<FArr> mask, uint32_t cachedTokens, uint32_t numHeads,
           uint32_t headDim, uint32_t latentDim, float scale) {
            if (Q.ndim() < 2) throw std::runtime_error("Q must be at least 2D");
            uint32_t B = 1, S = 1;
            if (Q.ndim() == 4) { B = uint32_t(Q.shape(0)); S = uint32_t(Q.shape(2)); }
            else if (Q.ndim() == 3) { B = uint32_t(Q.shape(0)); S = uint32_t(Q.shape(1)); }
            else S = uint32_t(Q.shape(0));
            if (size_t(Q.size()) != size_t(B) * numHeads * S * headDim)
                throw std::runtime_error("Q does not hold batch * num_heads * seq_len * head_dim values");
            if (size_t(latents.size()) < size_t(cachedTokens) * numHeads * latentDim)
                throw std::runtime_error("latents must hold cached_tokens * num_heads * latent_dim values");
            if (size_t(wUp.size()) != size_t(latentDim) * 2 * headDim)
                throw std::runtime_error("w_up must be (latent_dim, 2 * head_dim)");
            if (mask.has_value() && size_t(mask->size()) != size_t(B) * S * cachedTokens)
                throw std::runtime_error("mask must be (batch, seq_len, cached_tokens)");
            py::array_t<float> out({py::ssize_t(B), py::ssize_t(numHeads), py::ssize_t(S), py::ssize_t(headDim)});
            experimental::fusedAttentionCPU(Q.data(), latents.data(), wUp.data(), mask.has_value() ? mask->data() : nullptr,
                                            out.mutable_data(), B, S, cachedTokens, numHeads, headDim, latentDim, scale);
            return out;
        },
        py::arg("Q"), py::arg("latents"), py::arg("w_up"), py::arg("mask") = py::none(), py::arg("cached_tokens") = 0,
        py::arg("num_heads") = 8, py::arg("head_dim") = 64, py::arg("latent_dim") = 16, py::arg("scale") = 0.0f,
        "CPU reference for fused MLA decompression + attention.\n"
        "Decompresses latents via W_up matmul, then computes standard attention.");
    m.def(
        "kv_cache_set_mla_weights",
        [](GrillyCoreContext& ctx, ops::KVCache& kv, FArr wDown, FArr wUp) {
            const size_t n = size_t(2) * kv.config.headDim * kv.latentDim;
            if (!kv.mla() || size_t(wDown.size()) != n || size_t(wUp.size()) != n)
                throw std::runtime_error("kv_cache_set_mla_weights: w_down must be (2*head_dim, latent_dim) and w_up "
                                         "(latent_dim, 2*head_dim) of an MLA cache (compression_ratio > 1)");
            ops::kvCacheSetMLAWeights(ctx.pool, kv, wDown.data(), wUp.data());
        },
        py::arg("device"), py::arg("kv_cache"), py::arg("w_down"), py::arg("w_up"),
        "Set the MLA projection matrices (they start as zeros; the reference leaves them uninitialised)");
    m.def("kv_cache_latents", [](GrillyCoreContext& ctx, ops::KVCache& kv) {
        if (!kv.mla()) throw std::runtime_error("kv_cache_latents: not an MLA cache");
        const uint32_t T = kv.currentLen;
        py::array_t<float> out({py::ssize_t(T), py::ssize_t(kv.config.numHeads), py::ssize_t(kv.latentDim)});
        if (T) {
            check(grl_memcpy_d2h(ctx.device.handle(), out.mutable_data(), kv.latents.dptr, size_t(out.size()) * 4), "kv_cache_latents");
            check(grl_sync(ctx.device.handle(), 0), "kv_cache_latents");
        }
        return out;
    }, py::arg("device"), py::arg("kv_cache"), "Latents of an MLA cache: (tokens, heads, latent_dim) float32");
    // ---- linear projection (cpp/python/bindings.cpp:241-300 there) and the fused QKV projection
    m.def(
        "linear",
        [](GrillyCoreContext& ctx, FArr x, FArr weights, std::optional<FArr> bias, const std::string& dtype) {
            if (x.ndim() < 1 || x.ndim() > 3) throw std::runtime_error("x must be 1D, 2D, or 3D (batch, seq, input_dim)");
            if (weights.ndim() != 2) throw std::runtime_error("weights must be 2D (output_dim, input_dim)");
            const uint32_t inputDim = uint32_t(x.shape(x.ndim() - 1));
            const uint32_t batchSeq = uint32_t(size_t(x.size()) / std::max<uint32_t>(inputDim, 1));
            const uint32_t outputDim = uint32_t(weights.shape(0));
            if (uint32_t(weights.shape(1)) != inputDim)
                throw std::runtime_error("Weight input_dim mismatch: " + std::to_string(weights.shape(1)) + " vs " + std::to_string(inputDim));
            if (bias.has_value() && (bias->ndim() != 1 || uint32_t(bias->shape(0)) != outputDim))
                throw std::runtime_error("bias must be 1D with size output_dim");
            std::vector<py::ssize_t> shape;
            for (int i = 0; i + 1 < x.ndim(); ++i) shape.push_back(x.shape(i));
            if (x.ndim() == 1) shape.push_back(1);
            shape.push_back(outputDim);
            py::array_t<float> out(shape);
            ops::LinearParams p{batchSeq, inputDim, outputDim, bias.has_value() ? 1u : 0u};
            const float *xp = x.data(), *wp = weights.data(), *bp = bias.has_value() ? bias->data() : nullptr;
            float* op = out.mutable_data();
            const auto prec = parseDtype(dtype) == GRL_BF16 ? ops::Precision::BF16 : ops::Precision::FP32;
            {
                py::gil_scoped_release nogil;
                ops::linearEx(ctx.batch, ctx.pool, ctx.cache, xp, wp, bp, op, p, prec);
            }
            return out;
        },
        py::arg("device"), py::arg("x"), py::arg("weights"), py::arg("bias") = py::none(), py::arg("dtype") = "fp32",
        "GPU linear projection: output = x @ W^T + bias");
    m.def(
        "fused_qkv_projection",
        [](GrillyCoreContext& ctx, FArr x, FArr wQKV, std::optional<FArr> bQKV, uint32_t numHeads, uint32_t headDim,
           const std::string& dtype) {
            if (x.ndim() < 2 || x.ndim() > 3) throw std::runtime_error("x must be (batch_seq, hidden) or (batch, seq, hidden)");
            const uint32_t hidden = uint32_t(x.shape(x.ndim() - 1)), rows = uint32_t(size_t(x.size()) / hidden);
            const uint32_t qkv = 3 * numHeads * headDim;
            if (wQKV.ndim() != 2 || uint32_t(wQKV.shape(0)) != qkv || uint32_t(wQKV.shape(1)) != hidden)
                throw std::runtime_error("w_qkv must be (3 * num_heads * head_dim, hidden_dim): [W_q; W_k; W_v]");
            if (bQKV.has_value() && uint32_t(bQKV->size()) != qkv) throw std::runtime_error("b_qkv must hold 3 * num_heads * head_dim values");
            std::vector<py::ssize_t> shape;
            for (int i = 0; i + 1 < x.ndim(); ++i) shape.push_back(x.shape(i));
            shape.push_back(qkv);
            py::array_t<float> out(shape);
            const float *xp = x.data(), *wp = wQKV.data(), *bp = bQKV.has_value() ? bQKV->data() : nullptr;
            float* op = out.mutable_data();
            const auto prec = parseDtype(dtype) == GRL_BF16 ? ops::Precision::BF16 : ops::Precision::FP32;
            {
                py::gil_scoped_release nogil;
                ops::fusedQKVProjection(ctx.batch, ctx.pool, ctx.cache, xp, wp, bp, op, rows, hidden, numHeads, headDim, prec);
            }
            return out;
        },
        py::arg("device"), py::arg("x"), py::arg("w_qkv"), py::arg("b_qkv") = py::none(), py::arg("num_heads") = 8,
        py::arg("head_dim") = 64, py::arg("dtype") = "fp32",
        "Fused QKV projection: (batch_seq, hidden) -> (batch_seq, 3 * num_heads * head_dim) with [W_q; W_k; W_v]");
    for (const char* name : {"linear_cpu", "relu", "gelu", "silu", "tanh_act", "layernorm", "conv1d", "conv2d",
                             "hamming_search"})
        notBuilt(name, "outside the attention / KV-cache path that this CUDA build covers");
}

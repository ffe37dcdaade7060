// Drives include/infinicore_b200/ops.hpp (the C++ host layer over the C ABI) on inputs a Python test wrote:
//
//     infinicore_ops_test <dir>
//
// <dir>/manifest.txt lists tensors as `name dtype_code ndim d0 d1 ...` (raw contiguous bytes in <dir>/<name>.bin)
// and scalars as `scalar name value`.  The program uploads them, runs every wrapper (each twice, so the second
// call must be served from the descriptor cache), replays the two-call decode step from a captured graph,
// exercises eviction and error reporting, and writes results to <dir>/<name>.out.bin plus <dir>/report.txt.
// The Python side checks the results against the CPU oracle.
#include "infinicore_b200/ops.hpp"

#include <cstdio>
#include <fstream>
#include <iostream>
#include <map>
#include <sstream>
#include <string>
#include <thread>
#include <vector>

namespace ib = infinicore_b200;

namespace {

struct Blob {
    infiniDtype_t dtype;
    std::vector<size_t> shape;
    std::vector<char> host;
    void *device = nullptr;
    size_t bytes() const { return host.size(); }
};

size_t elemSize(infiniDtype_t dt) {
    switch (dt) {
    case INFINI_DTYPE_F16:
    case INFINI_DTYPE_BF16:
        return 2;
    case INFINI_DTYPE_F32:
    case INFINI_DTYPE_I32:
        return 4;
    default:
        return 8; // I64 / F64
    }
}

std::map<std::string, Blob> g_blobs;
std::map<std::string, double> g_scalars;
std::string g_dir;

void load(const std::string &dir) {
    std::ifstream manifest(dir + "/manifest.txt");
    if (!manifest) {
        throw std::runtime_error("no manifest.txt in " + dir);
    }
    std::string line;
    while (std::getline(manifest, line)) {
        std::istringstream in(line);
        std::string name;
        in >> name;
        if (name.empty()) {
            continue;
        }
        if (name == "scalar") {
            std::string key;
            double value;
            in >> key >> value;
            g_scalars[key] = value;
            continue;
        }
        int dtype, ndim;
        in >> dtype >> ndim;
        Blob b;
        b.dtype = static_cast<infiniDtype_t>(dtype);
        size_t count = 1;
        for (int i = 0; i < ndim; ++i) {
            size_t d;
            in >> d;
            b.shape.push_back(d);
            count *= d;
        }
        b.host.resize(count * elemSize(b.dtype));
        std::ifstream data(dir + "/" + name + ".bin", std::ios::binary);
        data.read(b.host.data(), static_cast<std::streamsize>(b.host.size()));
        if (static_cast<size_t>(data.gcount()) != b.host.size()) {
            throw std::runtime_error("short read of " + name);
        }
        ib::check(infinirtMalloc(&b.device, b.host.size() ? b.host.size() : 16), "infinirtMalloc");
        ib::check(infinirtMemcpy(b.device, b.host.data(), b.host.size(), INFINIRT_MEMCPY_H2D), "infinirtMemcpy");
        g_blobs[name] = std::move(b);
    }
}

ib::Tensor T(const std::string &name) {
    Blob &b = g_blobs.at(name);
    return ib::Tensor(b.device, b.dtype, b.shape);
}

// A fresh device copy of a loaded tensor (so scenarios do not see each other's cache updates).
ib::Tensor copyOf(const std::string &name, const std::string &as) {
    Blob b = g_blobs.at(name);
    b.device = nullptr;
    ib::check(infinirtMalloc(&b.device, b.bytes()), "infinirtMalloc");
    ib::check(infinirtMemcpy(b.device, b.host.data(), b.bytes(), INFINIRT_MEMCPY_H2D), "infinirtMemcpy");
    g_blobs[as] = std::move(b);
    return T(as);
}

// A zero-filled device tensor registered under `name`.
ib::Tensor zeros(const std::string &name, infiniDtype_t dtype, std::vector<size_t> shape) {
    Blob b;
    b.dtype = dtype;
    b.shape = std::move(shape);
    size_t count = 1;
    for (size_t d : b.shape) {
        count *= d;
    }
    b.host.assign(count * elemSize(dtype), 0);
    ib::check(infinirtMalloc(&b.device, b.bytes()), "infinirtMalloc");
    ib::check(infinirtMemcpy(b.device, b.host.data(), b.bytes(), INFINIRT_MEMCPY_H2D), "infinirtMemcpy");
    g_blobs[name] = std::move(b);
    return T(name);
}

void save(const std::string &name) {
    Blob &b = g_blobs.at(name);
    ib::check(infinirtDeviceSynchronize(), "infinirtDeviceSynchronize");
    ib::check(infinirtMemcpy(b.host.data(), b.device, b.bytes(), INFINIRT_MEMCPY_D2H), "infinirtMemcpy");
    std::ofstream out(g_dir + "/" + name + ".out.bin", std::ios::binary);
    out.write(b.host.data(), static_cast<std::streamsize>(b.bytes()));
}

} // namespace

int main(int argc, char **argv) {
    if (argc < 2) {
        std::fprintf(stderr, "usage: %s <dir>\n", argv[0]);
        return 2;
    }
    g_dir = argv[1];
    std::ofstream report;
    try {
        ib::check(infinirtSetDevice(INFINI_DEVICE_NVIDIA, 0), "infinirtSetDevice");
        load(g_dir);
        report.open(g_dir + "/report.txt");
        const float scale = static_cast<float>(g_scalars.at("scale"));
        const ib::Tensor q = T("q"), new_k = T("new_k"), new_v = T("new_v"), slots = T("slot_mapping"), tables = T("block_tables"),
                         lens = T("seq_lens");
        const std::vector<size_t> out_shape = {q.shape[0], q.shape[1], g_blobs.at("v_cache").shape[3]};
        const infiniDtype_t dt = q.dtype;

        // A. the reference's call sequence: paged_caching_ then paged_attention_, each twice
        {
            const ib::Tensor kc = copyOf("k_cache", "k_cache_a"), vc = copyOf("v_cache", "v_cache_a"), out = zeros("out_a", dt, out_shape);
            const ib::CacheStats before = ib::cache_stats();
            for (int i = 0; i < 2; ++i) {
                ib::op::paged_caching_(kc, vc, new_k, new_v, slots);
                ib::op::paged_attention_(out, q, kc, vc, tables, lens, std::nullopt, scale);
            }
            const ib::CacheStats after = ib::cache_stats();
            report << "two_call_misses " << after.misses - before.misses << "\n";
            report << "two_call_hits " << after.hits - before.hits << "\n";
            save("out_a"), save("k_cache_a"), save("v_cache_a");
        }
        // B. the same layer behind one call
        {
            const ib::Tensor kc = copyOf("k_cache", "k_cache_b"), vc = copyOf("v_cache", "v_cache_b"), out = zeros("out_b", dt, out_shape);
            ib::op::paged_decode_step_(out, q, kc, vc, new_k, new_v, tables, lens, std::nullopt, scale);
            save("out_b"), save("k_cache_b"), save("v_cache_b");
        }
        // C. ... with the rotary embedding of q and new_k in front, and D. the rotary embedding alone
        {
            const ib::Tensor kc = copyOf("k_cache", "k_cache_c"), vc = copyOf("v_cache", "v_cache_c"), out = zeros("out_c", dt, out_shape);
            ib::op::RotaryArgs rotary{T("pos_ids"), T("sin_table"), T("cos_table"), INFINIOP_ROPE_ALGO_GPT_NEOX};
            ib::op::paged_decode_step_(out, q, kc, vc, new_k, new_v, tables, lens, std::nullopt, scale, rotary);
            save("out_c"), save("k_cache_c"), save("v_cache_c");
            const ib::Tensor q_rot = zeros("q_rot", dt, q.shape);
            ib::op::rope_(q_rot, q, rotary.pos_ids, rotary.sin_table, rotary.cos_table, rotary.algo);
            save("q_rot");
        }
        // E. contiguous cache append
        {
            const ib::Tensor kc = copyOf("kvc_k_cache", "kvc_k_cache_e"), vc = copyOf("kvc_v_cache", "kvc_v_cache_e");
            ib::op::kv_caching_(kc, vc, T("kvc_k"), T("kvc_v"), T("kvc_past"));
            save("kvc_k_cache_e"), save("kvc_v_cache_e");
        }
        // F. prefill
        {
            const ib::Tensor pq = T("pf_q");
            const ib::Tensor out = zeros("out_pf", pq.dtype, {pq.shape[0], pq.shape[1], g_blobs.at("pf_v_cache").shape[3]});
            ib::op::paged_attention_prefill_(out, pq, T("pf_k_cache"), T("pf_v_cache"), T("pf_block_tables"), T("pf_seq_lens"), T("pf_cum"),
                                             std::nullopt, static_cast<float>(g_scalars.at("pf_scale")));
            save("out_pf");
        }
        // G. the two-call step captured into a graph on a stream of its own and replayed twice
        {
            const ib::Tensor kc = copyOf("k_cache", "k_cache_g"), vc = copyOf("v_cache", "v_cache_g"), out = zeros("out_g", dt, out_shape);
            infinirtStream_t stream = nullptr;
            ib::check(infinirtStreamCreate(&stream), "infinirtStreamCreate");
            // warm-up on this stream: descriptors exist, the stream's workspace is allocated
            ib::op::paged_caching_(kc, vc, new_k, new_v, slots, stream);
            ib::op::paged_attention_(out, q, kc, vc, tables, lens, std::nullopt, scale, stream);
            ib::check(infinirtStreamSynchronize(stream), "infinirtStreamSynchronize");
            ib::check(infinirtMemcpy(out.data, g_blobs.at("out_g").host.data(), g_blobs.at("out_g").bytes(), INFINIRT_MEMCPY_H2D), "infinirtMemcpy");
            const ib::CacheStats before = ib::cache_stats();
            infinirtGraph_t graph = nullptr;
            infinirtGraphExec_t exec = nullptr;
            ib::check(infinirtStreamBeginCapture(stream, INFINIRT_STREAM_CAPTURE_MODE_GLOBAL), "infinirtStreamBeginCapture");
            ib::op::paged_caching_(kc, vc, new_k, new_v, slots, stream);
            ib::op::paged_attention_(out, q, kc, vc, tables, lens, std::nullopt, scale, stream);
            ib::check(infinirtStreamEndCapture(stream, &graph), "infinirtStreamEndCapture");
            ib::check(infinirtGraphInstantiate(&exec, graph, nullptr, nullptr, 0), "infinirtGraphInstantiate");
            const ib::CacheStats after = ib::cache_stats();
            report << "capture_misses " << after.misses - before.misses << "\n";
            // a later, larger problem on this stream makes its workspace grow: the buffer the graph captured must
            // stay valid (it is retired, not freed), so the replays below still see their own scratch
            void *captured_ws = ib::detail::state().workspace(1, stream);
            void *grown_ws = ib::detail::state().workspace(static_cast<size_t>(96) << 20, stream);
            report << "workspace_moved " << (grown_ws != captured_ws ? 1 : 0) << "\n";
            ib::check(infinirtMemsetAsync(grown_ws, 0xff, static_cast<size_t>(96) << 20, stream), "infinirtMemsetAsync");
            for (int i = 0; i < 2; ++i) {
                ib::check(infinirtGraphLuanch(exec, stream), "infinirtGraphLuanch");
            }
            ib::check(infinirtStreamSynchronize(stream), "infinirtStreamSynchronize");
            save("out_g");
            ib::check(infinirtGraphExecDestroy(exec), "infinirtGraphExecDestroy");
            ib::check(infinirtGraphDestroy(graph), "infinirtGraphDestroy");
            ib::check(infinirtStreamDestroy(stream), "infinirtStreamDestroy");
        }
        // H. more distinct descriptors than the cache holds: the oldest are destroyed, the count stays bounded
        {
            const ib::CacheStats before = ib::cache_stats();
            const size_t rounds = ib::kDescriptorCacheCapacity + 10;
            for (size_t i = 0; i < rounds; ++i) {
                const size_t half = i + 1;
                ib::Tensor x(q.data, dt, {1, 1, 2 * half});
                ib::Tensor table(g_blobs.at("sin_table").device, dt, {1, half});
                ib::Tensor pos(g_blobs.at("pos_ids").device, g_blobs.at("pos_ids").dtype, {1});
                ib::Tensor y(g_blobs.at("q_rot").device, dt, {1, 1, 2 * half});
                ib::op::rope_(y, x, pos, table, table, INFINIOP_ROPE_ALGO_GPT_J);
            }
            ib::check(infinirtDeviceSynchronize(), "infinirtDeviceSynchronize");
            const ib::CacheStats after = ib::cache_stats();
            report << "evictions " << after.evictions - before.evictions << "\n";
            report << "cached " << ib::cached_descriptors() << "\n";
            report << "capacity " << ib::kDescriptorCacheCapacity << "\n";
        }
        // J. two more host threads at once, each with its own handle, descriptor cache, stream and workspace
        //    (the layer's state is per thread; libinfinirt's current device is too, so each thread selects it)
        {
            struct Job {
                ib::Tensor kc, vc, out;
                std::string error;
            };
            Job jobs[2];
            for (int t = 0; t < 2; ++t) {
                const std::string tag = "_j" + std::to_string(t);
                jobs[t].kc = copyOf("k_cache", "k_cache" + tag);
                jobs[t].vc = copyOf("v_cache", "v_cache" + tag);
                jobs[t].out = zeros("out" + tag, dt, out_shape);
            }
            auto work = [&](Job *job) {
                try {
                    ib::check(infinirtSetDevice(INFINI_DEVICE_NVIDIA, 0), "infinirtSetDevice");
                    infinirtStream_t stream = nullptr;
                    ib::check(infinirtStreamCreate(&stream), "infinirtStreamCreate");
                    for (int i = 0; i < 20; ++i) {
                        ib::op::paged_caching_(job->kc, job->vc, new_k, new_v, slots, stream);
                        ib::op::paged_attention_(job->out, q, job->kc, job->vc, tables, lens, std::nullopt, scale, stream);
                    }
                    ib::check(infinirtStreamSynchronize(stream), "infinirtStreamSynchronize");
                    if (ib::cache_stats().misses != 2) {
                        job->error = "a thread's cache should have missed exactly twice";
                    }
                    ib::clear_cache();
                    ib::check(infinirtStreamDestroy(stream), "infinirtStreamDestroy");
                } catch (const std::exception &e) {
                    job->error = e.what();
                }
            };
            std::thread a(work, &jobs[0]), b(work, &jobs[1]);
            a.join();
            b.join();
            for (int t = 0; t < 2; ++t) {
                if (!jobs[t].error.empty()) {
                    throw std::runtime_error("thread " + std::to_string(t) + ": " + jobs[t].error);
                }
                save("out_j" + std::to_string(t));
            }
            report << "threads 2\n";
        }
        // I. a rejected call surfaces as an exception carrying the status
        try {
            ib::Tensor wrong = T("new_v");
            wrong.dtype = INFINI_DTYPE_F32;
            ib::op::paged_caching_(T("k_cache_a"), T("v_cache_a"), new_k, wrong, slots);
            report << "error_status none\n";
        } catch (const ib::StatusError &e) {
            report << "error_status " << static_cast<int>(e.status) << "\n";
        }
        ib::clear_cache();
        report << "kernel_status " << ib::kernel_status() << "\n";
        report << "cached_after_clear " << ib::cached_descriptors() << "\n";
        report << "ok 1\n";
    } catch (const std::exception &e) {
        std::fprintf(stderr, "infinicore_ops_test: %s\n", e.what());
        return 1;
    }
    return 0;
}

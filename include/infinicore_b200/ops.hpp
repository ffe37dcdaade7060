// C++ host layer over the C ABI of libinfiniop / libinfinirt for the paged decode path: the counterpart of
// the reference's infinicore operator layer for these operators
// (src/infinicore/ops/paged_attention/paged_attention_infiniop.cc:47-64,
//  src/infinicore/ops/paged_caching/paged_caching_infiniop.cc:38-51, src/infinicore/ops/infiniop_impl.hpp:8-73).
//
// What the reference's layer does for a caller, and this header does too:
//   * one infiniop handle per (thread, device), created on first use for the thread's current device
//     (reference src/infinicore/context: the current device is thread-local, as in libinfinirt);
//   * operator descriptors cached per (thread, device), least recently used evicted (the reference keeps 100
//     per operator, infiniop_impl.hpp:43-48; here one cache of `kDescriptorCacheCapacity` entries is shared
//     by all operators and keyed by the exact tensor metadata, not by a hash of it);
//   * a workspace per (thread, device, stream), grown on demand (the reference allocates a workspace tensor per
//     call, infiniop_impl.hpp:66-73; a grow-only buffer keeps the calls allocation-free, which CUDA-graph
//     capture needs);
//   * status codes turned into exceptions (INFINICORE_CHECK_ERROR).
//
// Header-only, C++17, no CUDA headers needed: tensors are non-owning views of device memory.  Functions ending
// in an underscore write into their first argument, like the reference's `paged_attention_` / `paged_caching_`.
#ifndef INFINICORE_B200_OPS_HPP
#define INFINICORE_B200_OPS_HPP

#include "../infiniop.h"
#include "../infinirt.h"

#include <cstddef>
#include <cstring>
#include <list>
#include <map>
#include <optional>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

namespace infinicore_b200 {

// A non-owning view of device memory; strides in elements.
struct Tensor {
    void *data = nullptr;
    infiniDtype_t dtype = INFINI_DTYPE_INVALID;
    std::vector<size_t> shape;
    std::vector<ptrdiff_t> strides;

    Tensor() = default;
    // contiguous view
    Tensor(void *data_, infiniDtype_t dtype_, std::vector<size_t> shape_) : data(data_), dtype(dtype_), shape(std::move(shape_)) {
        strides.assign(shape.size(), 1);
        ptrdiff_t run = 1;
        for (size_t i = shape.size(); i-- > 0;) {
            strides[i] = run;
            run *= static_cast<ptrdiff_t>(shape[i]);
        }
    }
    Tensor(void *data_, infiniDtype_t dtype_, std::vector<size_t> shape_, std::vector<ptrdiff_t> strides_)
        : data(data_), dtype(dtype_), shape(std::move(shape_)), strides(std::move(strides_)) {}
};

class StatusError : public std::runtime_error {
public:
    StatusError(infiniStatus_t status_, const char *what_)
        : std::runtime_error(std::string(what_) + " failed with infiniStatus_t " + std::to_string(static_cast<int>(status_))), status(status_) {}
    infiniStatus_t status;
};

inline void check(infiniStatus_t status, const char *what) {
    if (status != INFINI_STATUS_SUCCESS) {
        throw StatusError(status, what);
    }
}

constexpr size_t kDescriptorCacheCapacity = 256;

struct CacheStats {
    size_t hits = 0;
    size_t misses = 0;
    size_t evictions = 0;
};

namespace detail {

// Owns one tensor descriptor for the duration of an operator-descriptor creation (the operator descriptor
// copies what it needs, so the tensor descriptors go away right after).
class TensorDesc {
public:
    explicit TensorDesc(const Tensor *t) {
        if (t != nullptr) {
            check(infiniopCreateTensorDescriptor(&desc_, t->shape.size(), t->shape.data(), t->strides.data(), t->dtype),
                  "infiniopCreateTensorDescriptor");
        }
    }
    TensorDesc(const TensorDesc &) = delete;
    TensorDesc &operator=(const TensorDesc &) = delete;
    ~TensorDesc() {
        if (desc_ != nullptr) {
            infiniopDestroyTensorDescriptor(desc_);
        }
    }
    infiniopTensorDescriptor_t get() const { return desc_; }

private:
    infiniopTensorDescriptor_t desc_ = nullptr;
};

// Exact cache key: an operator tag followed by the raw metadata of every tensor and scalar that the
// descriptor depends on.
class Key {
public:
    explicit Key(const char *op) { bytes_.assign(op); bytes_.push_back('\0'); }
    Key &add(const Tensor *t) {
        if (t == nullptr) {
            bytes_.push_back('-');
            return *this;
        }
        raw(static_cast<int>(t->dtype));
        raw(t->shape.size());
        for (size_t d : t->shape) {
            raw(d);
        }
        for (ptrdiff_t s : t->strides) {
            raw(s);
        }
        return *this;
    }
    template <typename V>
    Key &raw(const V &v) {
        const char *p = reinterpret_cast<const char *>(&v);
        bytes_.append(p, sizeof(V));
        return *this;
    }
    const std::string &str() const { return bytes_; }

private:
    std::string bytes_;
};

struct Entry {
    InfiniopDescriptor *desc = nullptr;
    size_t workspace_bytes = 0;
    infiniStatus_t (*destroy)(InfiniopDescriptor *) = nullptr;
};

class LruCache {
public:
    explicit LruCache(size_t capacity) : capacity_(capacity) {}
    LruCache(const LruCache &) = delete;
    LruCache &operator=(const LruCache &) = delete;
    ~LruCache() { clear(); }

    const Entry *get(const std::string &key) {
        auto it = index_.find(key);
        if (it == index_.end()) {
            ++stats.misses;
            return nullptr;
        }
        order_.splice(order_.begin(), order_, it->second); // most recently used first
        ++stats.hits;
        return &it->second->second;
    }

    const Entry *put(const std::string &key, const Entry &entry) {
        while (!order_.empty() && order_.size() >= capacity_) {
            release(order_.back().second);
            index_.erase(order_.back().first);
            order_.pop_back();
            ++stats.evictions;
        }
        order_.emplace_front(key, entry);
        index_[key] = order_.begin();
        return &order_.front().second;
    }

    void clear() {
        for (auto &kv : order_) {
            release(kv.second);
        }
        order_.clear();
        index_.clear();
    }

    size_t size() const { return order_.size(); }
    CacheStats stats;

private:
    static void release(Entry &e) {
        if (e.desc != nullptr && e.destroy != nullptr) {
            e.destroy(e.desc);
            e.desc = nullptr;
        }
    }
    size_t capacity_;
    std::list<std::pair<std::string, Entry>> order_;
    std::unordered_map<std::string, std::list<std::pair<std::string, Entry>>::iterator> index_;
};

struct Workspace {
    void *ptr = nullptr;
    size_t bytes = 0;
};

// Everything one thread keeps for one device.
struct DeviceState {
    explicit DeviceState(int device_id_) : device_id(device_id_), cache(kDescriptorCacheCapacity) {
        check(infiniopCreateHandle(&handle), "infiniopCreateHandle");
    }
    DeviceState(const DeviceState &) = delete;
    DeviceState &operator=(const DeviceState &) = delete;
    ~DeviceState() {
        cache.clear();
        for (auto &kv : workspaces) {
            if (kv.second.ptr != nullptr) {
                infinirtFree(kv.second.ptr);
            }
        }
        for (void *old : retired) {
            infinirtFree(old);
        }
        if (handle != nullptr) {
            infiniopDestroyHandle(handle);
        }
    }

    // Grow-only scratch per stream.  A buffer that a larger request supersedes is not freed but kept until this
    // state dies: kernels in flight, and CUDA graphs captured earlier, may still hold its address.  Steady-state
    // calls never allocate, which stream capture needs; run the largest problem of a stream once BEFORE
    // capturing on it, because growing means infinirtMalloc, and that is not allowed inside a capture.
    void *workspace(size_t bytes, infinirtStream_t stream) {
        if (bytes == 0) {
            return nullptr;
        }
        Workspace &w = workspaces[stream];
        if (w.bytes < bytes) {
            void *fresh = nullptr;
            check(infinirtMalloc(&fresh, bytes), "infinirtMalloc");
            if (w.ptr != nullptr) {
                retired.push_back(w.ptr);
            }
            w.ptr = fresh;
            w.bytes = bytes;
        }
        return w.ptr;
    }

    int device_id;
    infiniopHandle_t handle = nullptr;
    LruCache cache;
    std::map<infinirtStream_t, Workspace> workspaces;
    std::vector<void *> retired; // superseded workspaces, freed with the state
};

// The calling thread's state for its current device (libinfinirt's current device is thread-local and
// infiniopCreateHandle binds to it).
inline DeviceState &state() {
    thread_local std::map<int, DeviceState> states;
    infiniDevice_t device = INFINI_DEVICE_NVIDIA;
    int device_id = 0;
    check(infinirtGetDevice(&device, &device_id), "infinirtGetDevice");
    if (device != INFINI_DEVICE_NVIDIA) {
        // a thread that never selected a device: take NVIDIA device 0, as the reference's context does for its default
        check(infinirtSetDevice(INFINI_DEVICE_NVIDIA, 0), "infinirtSetDevice");
        device_id = 0;
    }
    auto it = states.find(device_id);
    if (it == states.end()) {
        it = states.try_emplace(device_id, device_id).first;
    }
    return it->second;
}

template <typename Create, typename WorkspaceSize>
inline const Entry &lookup(DeviceState &st, const Key &key, Create create, WorkspaceSize workspace_size,
                           infiniStatus_t (*destroy)(InfiniopDescriptor *), const char *what) {
    if (const Entry *hit = st.cache.get(key.str())) {
        return *hit;
    }
    Entry e;
    e.destroy = destroy;
    check(create(st.handle, &e.desc), what);
    const infiniStatus_t ws = workspace_size(e.desc, &e.workspace_bytes);
    if (ws != INFINI_STATUS_SUCCESS) {
        destroy(e.desc);
        throw StatusError(ws, what);
    }
    return *st.cache.put(key.str(), e);
}

} // namespace detail

// Hit / miss / eviction counts of the calling thread's descriptor cache for its current device.
inline CacheStats cache_stats() { return detail::state().cache.stats; }
inline size_t cached_descriptors() { return detail::state().cache.size(); }
// Destroys the calling thread's cached descriptors for its current device.
inline void clear_cache() { detail::state().cache.clear(); }

// Waits for `stream`, returns the current device's word of kernel status flags and clears it
// (include/infiniop/ops/kernel_status.h): 0 when every kernel of the library did all of its work.
inline unsigned int kernel_status(infinirtStream_t stream = nullptr) {
    unsigned int flags = 0;
    check(infiniopGetKernelStatus(detail::state().handle, stream, &flags), "infiniopGetKernelStatus");
    return flags;
}

namespace op {

namespace detail_op {
inline const Tensor *ptr(const std::optional<Tensor> &t) { return t.has_value() ? &*t : nullptr; }
inline const void *data(const std::optional<Tensor> &t) { return t.has_value() ? t->data : nullptr; }
} // namespace detail_op

// out [seqs, heads, value] = decode attention of q [seqs, heads, head] over the paged cache
// (reference include/infinicore/ops/paged_attention.hpp:16-18).
inline void paged_attention_(const Tensor &out, const Tensor &q, const Tensor &k_cache, const Tensor &v_cache, const Tensor &block_tables,
                             const Tensor &kv_lens, const std::optional<Tensor> &alibi_slopes, float scale, infinirtStream_t stream = nullptr) {
    using namespace detail;
    DeviceState &st = state();
    const Tensor *alibi = detail_op::ptr(alibi_slopes);
    Key key("paged_attention");
    key.add(&out).add(&q).add(&k_cache).add(&v_cache).add(&block_tables).add(&kv_lens).add(alibi).raw(scale);
    const Entry &e = lookup(
        st, key,
        [&](infiniopHandle_t h, InfiniopDescriptor **d) {
            TensorDesc o(&out), tq(&q), kc(&k_cache), vc(&v_cache), bt(&block_tables), sl(&kv_lens), al(alibi);
            return infiniopCreatePagedAttentionDescriptor(h, d, o.get(), tq.get(), kc.get(), vc.get(), bt.get(), sl.get(), al.get(), scale);
        },
        infiniopGetPagedAttentionWorkspaceSize, infiniopDestroyPagedAttentionDescriptor, "infiniopCreatePagedAttentionDescriptor");
    check(infiniopPagedAttention(e.desc, st.workspace(e.workspace_bytes, stream), e.workspace_bytes, out.data, q.data, k_cache.data,
                                 v_cache.data, block_tables.data, kv_lens.data, detail_op::data(alibi_slopes), stream),
          "infiniopPagedAttention");
}

// Scatter of k / v [tokens, kv_heads, head] into the pools at slot_mapping (reference include/infinicore/ops/paged_caching.hpp).
inline void paged_caching_(const Tensor &k_cache, const Tensor &v_cache, const Tensor &k, const Tensor &v, const Tensor &slot_mapping,
                           infinirtStream_t stream = nullptr) {
    using namespace detail;
    DeviceState &st = state();
    Key key("paged_caching");
    key.add(&k_cache).add(&v_cache).add(&k).add(&v).add(&slot_mapping);
    const Entry &e = lookup(
        st, key,
        [&](infiniopHandle_t h, InfiniopDescriptor **d) {
            TensorDesc kc(&k_cache), vc(&v_cache), tk(&k), tv(&v), sm(&slot_mapping);
            return infiniopCreatePagedCachingDescriptor(h, d, kc.get(), vc.get(), tk.get(), tv.get(), sm.get());
        },
        infiniopGetPagedCachingWorkspaceSize, infiniopDestroyPagedCachingDescriptor, "infiniopCreatePagedCachingDescriptor");
    check(infiniopPagedCaching(e.desc, st.workspace(e.workspace_bytes, stream), e.workspace_bytes, k_cache.data, v_cache.data, k.data,
                               v.data, slot_mapping.data, stream),
          "infiniopPagedCaching");
}

// Causal attention of packed new tokens q [total_q, heads, head] over the paged cache that already holds them.
inline void paged_attention_prefill_(const Tensor &out, const Tensor &q, const Tensor &k_cache, const Tensor &v_cache,
                                     const Tensor &block_tables, const Tensor &kv_lens, const Tensor &cum_seq_lens_q,
                                     const std::optional<Tensor> &alibi_slopes, float scale, infinirtStream_t stream = nullptr) {
    using namespace detail;
    DeviceState &st = state();
    const Tensor *alibi = detail_op::ptr(alibi_slopes);
    Key key("paged_attention_prefill");
    key.add(&out).add(&q).add(&k_cache).add(&v_cache).add(&block_tables).add(&kv_lens).add(&cum_seq_lens_q).add(alibi).raw(scale);
    const Entry &e = lookup(
        st, key,
        [&](infiniopHandle_t h, InfiniopDescriptor **d) {
            TensorDesc o(&out), tq(&q), kc(&k_cache), vc(&v_cache), bt(&block_tables), sl(&kv_lens), cq(&cum_seq_lens_q), al(alibi);
            return infiniopCreatePagedAttentionPrefillDescriptor(h, d, o.get(), tq.get(), kc.get(), vc.get(), bt.get(), sl.get(), cq.get(),
                                                                 al.get(), scale);
        },
        infiniopGetPagedAttentionPrefillWorkspaceSize, infiniopDestroyPagedAttentionPrefillDescriptor,
        "infiniopCreatePagedAttentionPrefillDescriptor");
    check(infiniopPagedAttentionPrefill(e.desc, st.workspace(e.workspace_bytes, stream), e.workspace_bytes, out.data, q.data, k_cache.data,
                                        v_cache.data, block_tables.data, kv_lens.data, cum_seq_lens_q.data, detail_op::data(alibi_slopes),
                                        stream),
          "infiniopPagedAttentionPrefill");
}

// Rotary embedding; y may be x (reference include/infinicore/ops/rope.hpp).
inline void rope_(const Tensor &y, const Tensor &x, const Tensor &pos_ids, const Tensor &sin_table, const Tensor &cos_table,
                  infiniopRoPEAlgo_t algo, infinirtStream_t stream = nullptr) {
    using namespace detail;
    DeviceState &st = state();
    Key key("rope");
    key.add(&y).add(&x).add(&pos_ids).add(&sin_table).add(&cos_table).raw(static_cast<int>(algo));
    const Entry &e = lookup(
        st, key,
        [&](infiniopHandle_t h, InfiniopDescriptor **d) {
            TensorDesc ty(&y), tx(&x), tp(&pos_ids), ts(&sin_table), tc(&cos_table);
            return infiniopCreateRoPEDescriptor(h, d, ty.get(), tx.get(), tp.get(), ts.get(), tc.get(), algo);
        },
        infiniopGetRoPEWorkspaceSize, infiniopDestroyRoPEDescriptor, "infiniopCreateRoPEDescriptor");
    check(infiniopRoPE(e.desc, st.workspace(e.workspace_bytes, stream), e.workspace_bytes, y.data, x.data, pos_ids.data, sin_table.data,
                       cos_table.data, stream),
          "infiniopRoPE");
}

// Append to a contiguous cache [batch, kv_heads, max_seq_len, hidden] (reference include/infinicore/ops/kv_caching.hpp).
inline void kv_caching_(const Tensor &k_cache, const Tensor &v_cache, const Tensor &k, const Tensor &v, const Tensor &past_kv_lengths,
                        infinirtStream_t stream = nullptr) {
    using namespace detail;
    DeviceState &st = state();
    Key key("kv_caching");
    key.add(&k_cache).add(&v_cache).add(&k).add(&v).add(&past_kv_lengths);
    const Entry &e = lookup(
        st, key,
        [&](infiniopHandle_t h, InfiniopDescriptor **d) {
            TensorDesc kc(&k_cache), vc(&v_cache), tk(&k), tv(&v), pl(&past_kv_lengths);
            return infiniopCreateKVCachingDescriptor(h, d, kc.get(), vc.get(), tk.get(), tv.get(), pl.get());
        },
        infiniopGetKVCachingWorkspaceSize, infiniopDestroyKVCachingDescriptor, "infiniopCreateKVCachingDescriptor");
    check(infiniopKVCaching(e.desc, st.workspace(e.workspace_bytes, stream), e.workspace_bytes, k_cache.data, v_cache.data, k.data, v.data,
                            past_kv_lengths.data, stream),
          "infiniopKVCaching");
}

// Position ids and tables for the RoPE form of the decode step.
struct RotaryArgs {
    Tensor pos_ids;   // [seqs], any integer type
    Tensor sin_table; // [table_len, head / 2]
    Tensor cos_table; // [table_len, head / 2]
    infiniopRoPEAlgo_t algo = INFINIOP_ROPE_ALGO_GPT_NEOX;
};

// One decode layer behind one call (no reference counterpart): append new_k / new_v [seqs, kv_heads, head] at
// position kv_lens[i] - 1 of every sequence, then attend.  With `rotary`, q and new_k are rotated first (the
// cache receives the rotated row; q and new_k themselves stay as they are).
inline void paged_decode_step_(const Tensor &out, const Tensor &q, const Tensor &k_cache, const Tensor &v_cache, const Tensor &new_k,
                               const Tensor &new_v, const Tensor &block_tables, const Tensor &kv_lens,
                               const std::optional<Tensor> &alibi_slopes, float scale, const std::optional<RotaryArgs> &rotary = std::nullopt,
                               infinirtStream_t stream = nullptr) {
    using namespace detail;
    DeviceState &st = state();
    const Tensor *alibi = detail_op::ptr(alibi_slopes);
    const RotaryArgs *r = rotary.has_value() ? &*rotary : nullptr;
    Key key(r != nullptr ? "paged_decode_step_rope" : "paged_decode_step");
    key.add(&out).add(&q).add(&k_cache).add(&v_cache).add(&new_k).add(&new_v).add(&block_tables).add(&kv_lens).add(alibi).raw(scale);
    if (r != nullptr) {
        key.add(&r->pos_ids).add(&r->sin_table).add(&r->cos_table).raw(static_cast<int>(r->algo));
    }
    const Entry &e = lookup(
        st, key,
        [&](infiniopHandle_t h, InfiniopDescriptor **d) {
            TensorDesc o(&out), tq(&q), kc(&k_cache), vc(&v_cache), nk(&new_k), nv(&new_v), bt(&block_tables), sl(&kv_lens), al(alibi);
            if (r == nullptr) {
                return infiniopCreatePagedDecodeStepDescriptor(h, d, o.get(), tq.get(), kc.get(), vc.get(), nk.get(), nv.get(), bt.get(),
                                                               sl.get(), al.get(), scale);
            }
            TensorDesc tp(&r->pos_ids), ts(&r->sin_table), tc(&r->cos_table);
            return infiniopCreatePagedDecodeStepRoPEDescriptor(h, d, o.get(), tq.get(), kc.get(), vc.get(), nk.get(), nv.get(), bt.get(),
                                                               sl.get(), al.get(), tp.get(), ts.get(), tc.get(), r->algo, scale);
        },
        infiniopGetPagedDecodeStepWorkspaceSize, infiniopDestroyPagedDecodeStepDescriptor, "infiniopCreatePagedDecodeStepDescriptor");
    void *ws = st.workspace(e.workspace_bytes, stream);
    if (r == nullptr) {
        check(infiniopPagedDecodeStep(e.desc, ws, e.workspace_bytes, out.data, q.data, k_cache.data, v_cache.data, new_k.data, new_v.data,
                                      block_tables.data, kv_lens.data, detail_op::data(alibi_slopes), stream),
              "infiniopPagedDecodeStep");
    } else {
        check(infiniopPagedDecodeStepRoPE(e.desc, ws, e.workspace_bytes, out.data, q.data, k_cache.data, v_cache.data, new_k.data,
                                          new_v.data, block_tables.data, kv_lens.data, detail_op::data(alibi_slopes), r->pos_ids.data,
                                          r->sin_table.data, r->cos_table.data, stream),
              "infiniopPagedDecodeStepRoPE");
    }
}

} // namespace op
} // namespace infinicore_b200

#endif

// C ABI plumbing: device, buffers, streams, events, transfers.
// Mirrors the handle and error conventions of backend/hip/bridge/bridge.cpp.
#include <cstring>

#include <cstdlib>

#include "common.cuh"

namespace yk {

std::string & last_error_ref() {
    static thread_local std::string msg;
    return msg;
}

yuuka_status fail(yuuka_status code, const char * fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    last_error_ref() = buf;
    return code;
}

}  // namespace yk

using namespace yk;

namespace yk {
bool pdl_enabled() {
    static const bool on = [] {
        const char * e = getenv("YUUKA_CUDA_NO_PDL");
        return !(e && e[0] == '1');
    }();
    return on;
}
}  // namespace yk

extern "C" {

uint32_t yuuka_abi_version(void) { return YUUKA_CUDA_ABI_VERSION; }

const char * yuuka_last_error(void) { return last_error_ref().c_str(); }

yuuka_status yuuka_device_open(int32_t index, yuuka_device ** out) {
    return guard([&] {
        YK_REQUIRE(out != nullptr, YUUKA_ERR_INVALID_ARGUMENT, "device_open: out is null");
        *out = nullptr;
        int count = 0;
        cudaError_t err = cudaGetDeviceCount(&count);
        YK_REQUIRE(err == cudaSuccess && count > 0, YUUKA_ERR_DEVICE,
                   "no CUDA device is available (%s); this library has no CPU fallback",
                   err == cudaSuccess ? "device count is zero" : cudaGetErrorString(err));
        YK_REQUIRE(index >= 0 && index < count, YUUKA_ERR_INVALID_ARGUMENT,
                   "device index %d is outside 0..%d", index, count - 1);
        auto * dev = new yuuka_device();
        dev->index = index;
        YK_CUDA(cudaSetDevice(index));
        YK_CUDA(cudaGetDeviceProperties(&dev->prop, index));
        dev->sm_count = dev->prop.multiProcessorCount;
        if (dev->prop.major < 10) {
            int major = dev->prop.major, minor = dev->prop.minor;
            delete dev;
            YK_REQUIRE(false, YUUKA_ERR_UNSUPPORTED,
                       "device is sm_%d%d; this library is built for sm_100a only", major, minor);
        }
        *out = dev;
    });
}

void yuuka_device_close(yuuka_device * dev) { delete dev; }

yuuka_status yuuka_device_info_get(const yuuka_device * dev, yuuka_device_info * info) {
    return guard([&] {
        YK_REQUIRE(dev && info, YUUKA_ERR_INVALID_ARGUMENT, "device_info_get: null argument");
        memset(info, 0, sizeof(*info));
        snprintf(info->name, sizeof(info->name), "%s", dev->prop.name);
        snprintf(info->arch, sizeof(info->arch), "sm_%d%d", dev->prop.major, dev->prop.minor);
        int rt = 0;
        cudaRuntimeGetVersion(&rt);
        snprintf(info->cuda_version, sizeof(info->cuda_version), "%d.%d", rt / 1000, (rt % 1000) / 10);
        info->total_memory = dev->prop.totalGlobalMem;
        info->multiprocessors = (uint32_t)dev->prop.multiProcessorCount;
        int khz = 0;
        cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev->index);
        info->clock_mhz = (uint32_t)(khz / 1000);
        info->l2_bytes = (uint32_t)dev->prop.l2CacheSize;
        info->smem_per_block_optin = (uint32_t)dev->prop.sharedMemPerBlockOptin;
        info->pci_domain = dev->prop.pciDomainID;
        info->pci_bus = dev->prop.pciBusID;
        info->pci_device = dev->prop.pciDeviceID;
    });
}

yuuka_status yuuka_device_memory_get(const yuuka_device * dev, uint64_t * free_bytes, uint64_t * total_bytes) {
    return guard([&] {
        YK_REQUIRE(dev && free_bytes && total_bytes, YUUKA_ERR_INVALID_ARGUMENT, "device_memory_get: null argument");
        set_device(dev);
        size_t f = 0, t = 0;
        YK_CUDA(cudaMemGetInfo(&f, &t));
        *free_bytes = f;
        *total_bytes = t;
    });
}

yuuka_status yuuka_buffer_alloc(yuuka_device * dev, uint64_t bytes, yuuka_buffer ** out) {
    return guard([&] {
        YK_REQUIRE(dev && out, YUUKA_ERR_INVALID_ARGUMENT, "buffer_alloc: null argument");
        *out = nullptr;
        YK_REQUIRE(bytes > 0, YUUKA_ERR_INVALID_ARGUMENT, "buffer_alloc: zero bytes");
        set_device(dev);
        void * ptr = nullptr;
        cudaError_t err = cudaMalloc(&ptr, bytes);
        if (err != cudaSuccess) {
            cudaGetLastError();
            YK_REQUIRE(false, YUUKA_ERR_ALLOCATION, "cudaMalloc(%llu) failed: %s",
                       (unsigned long long)bytes, cudaGetErrorString(err));
        }
        auto * buf = new yuuka_buffer();
        buf->dev = dev;
        buf->ptr = ptr;
        buf->bytes = bytes;
        *out = buf;
    });
}

void yuuka_buffer_free(yuuka_buffer * buf) {
    if (!buf) return;
    if (buf->ptr) {
        cudaSetDevice(buf->dev->index);
        cudaFree(buf->ptr);
    }
    delete buf;
}

uint64_t yuuka_buffer_size(const yuuka_buffer * buf) { return buf ? buf->bytes : 0; }
void * yuuka_buffer_ptr(const yuuka_buffer * buf) { return buf ? buf->ptr : nullptr; }

yuuka_status yuuka_stream_create(yuuka_device * dev, yuuka_stream ** out) {
    return guard([&] {
        YK_REQUIRE(dev && out, YUUKA_ERR_INVALID_ARGUMENT, "stream_create: null argument");
        *out = nullptr;
        set_device(dev);
        auto * s = new yuuka_stream();
        s->dev = dev;
        cudaError_t err = cudaStreamCreateWithFlags(&s->s, cudaStreamNonBlocking);
        if (err != cudaSuccess) {
            delete s;
            YK_CUDA(err);
        }
        *out = s;
    });
}

void yuuka_stream_destroy(yuuka_stream * stream) {
    if (!stream) return;
    if (stream->s) {
        cudaSetDevice(stream->dev->index);
        cudaStreamDestroy(stream->s);
    }
    delete stream;
}

yuuka_status yuuka_stream_synchronize(yuuka_stream * stream) {
    return guard([&] {
        YK_REQUIRE(stream, YUUKA_ERR_INVALID_ARGUMENT, "stream_synchronize: null stream");
        set_device(stream->dev);
        YK_CUDA(cudaStreamSynchronize(stream->s));
    });
}

yuuka_status yuuka_event_create(yuuka_device * dev, yuuka_event ** out) {
    return guard([&] {
        YK_REQUIRE(dev && out, YUUKA_ERR_INVALID_ARGUMENT, "event_create: null argument");
        *out = nullptr;
        set_device(dev);
        auto * e = new yuuka_event();
        e->dev = dev;
        cudaError_t err = cudaEventCreate(&e->e);
        if (err != cudaSuccess) {
            delete e;
            YK_CUDA(err);
        }
        *out = e;
    });
}

void yuuka_event_destroy(yuuka_event * event) {
    if (!event) return;
    if (event->e) {
        cudaSetDevice(event->dev->index);
        cudaEventDestroy(event->e);
    }
    delete event;
}

yuuka_status yuuka_event_record(yuuka_stream * stream, yuuka_event * event) {
    return guard([&] {
        YK_REQUIRE(stream && event, YUUKA_ERR_INVALID_ARGUMENT, "event_record: null argument");
        set_device(stream->dev);
        YK_CUDA(cudaEventRecord(event->e, stream->s));
    });
}

yuuka_status yuuka_event_wait(yuuka_event * event) {
    return guard([&] {
        YK_REQUIRE(event, YUUKA_ERR_INVALID_ARGUMENT, "event_wait: null event");
        set_device(event->dev);
        YK_CUDA(cudaEventSynchronize(event->e));
    });
}

yuuka_status yuuka_event_elapsed_ms(yuuka_event * start, yuuka_event * end, float * ms) {
    return guard([&] {
        YK_REQUIRE(start && end && ms, YUUKA_ERR_INVALID_ARGUMENT, "event_elapsed_ms: null argument");
        set_device(start->dev);
        YK_CUDA(cudaEventElapsedTime(ms, start->e, end->e));
    });
}

yuuka_status yuuka_memcpy_h2d_at(yuuka_buffer * dst, uint64_t offset, const void * src, uint64_t bytes) {
    return guard([&] {
        YK_REQUIRE(dst && src, YUUKA_ERR_INVALID_ARGUMENT, "memcpy_h2d: null argument");
        YK_REQUIRE(offset <= dst->bytes && bytes <= dst->bytes - offset, YUUKA_ERR_INVALID_ARGUMENT,
                   "memcpy_h2d: %llu bytes at offset %llu exceed the %llu-byte buffer",
                   (unsigned long long)bytes, (unsigned long long)offset, (unsigned long long)dst->bytes);
        if (bytes == 0) return;
        set_device(dst->dev);
        YK_CUDA(cudaMemcpy((char *)dst->ptr + offset, src, bytes, cudaMemcpyHostToDevice));
    });
}

yuuka_status yuuka_memcpy_h2d(yuuka_buffer * dst, const void * src, uint64_t bytes) {
    return yuuka_memcpy_h2d_at(dst, 0, src, bytes);
}

yuuka_status yuuka_memcpy_d2h_at(void * dst, const yuuka_buffer * src, uint64_t offset, uint64_t bytes) {
    return guard([&] {
        YK_REQUIRE(dst && src, YUUKA_ERR_INVALID_ARGUMENT, "memcpy_d2h: null argument");
        YK_REQUIRE(offset <= src->bytes && bytes <= src->bytes - offset, YUUKA_ERR_INVALID_ARGUMENT,
                   "memcpy_d2h: %llu bytes at offset %llu exceed the %llu-byte buffer",
                   (unsigned long long)bytes, (unsigned long long)offset, (unsigned long long)src->bytes);
        if (bytes == 0) return;
        set_device(src->dev);
        YK_CUDA(cudaMemcpy(dst, (const char *)src->ptr + offset, bytes, cudaMemcpyDeviceToHost));
    });
}

yuuka_status yuuka_memcpy_d2h(void * dst, const yuuka_buffer * src, uint64_t bytes) {
    return yuuka_memcpy_d2h_at(dst, src, 0, bytes);
}

yuuka_status yuuka_memset(yuuka_stream * stream, yuuka_buffer * dst, int value, uint64_t bytes) {
    return guard([&] {
        YK_REQUIRE(stream && dst, YUUKA_ERR_INVALID_ARGUMENT, "memset: null argument");
        YK_REQUIRE(bytes <= dst->bytes, YUUKA_ERR_INVALID_ARGUMENT, "memset: range exceeds the buffer");
        set_device(dst->dev);
        YK_CUDA(cudaMemsetAsync(dst->ptr, value, bytes, stream->s));
    });
}

yuuka_status yuuka_buffer_copy(yuuka_stream * stream, yuuka_buffer * dst, uint64_t dst_offset,
                               const yuuka_buffer * src, uint64_t src_offset, uint64_t bytes,
                               yuuka_event * completion) {
    return guard([&] {
        YK_REQUIRE(stream && dst && src, YUUKA_ERR_INVALID_ARGUMENT, "buffer_copy: null argument");
        YK_REQUIRE(dst_offset <= dst->bytes && bytes <= dst->bytes - dst_offset &&
                       src_offset <= src->bytes && bytes <= src->bytes - src_offset,
                   YUUKA_ERR_INVALID_ARGUMENT, "buffer_copy: range exceeds a buffer");
        set_device(dst->dev);
        if (bytes)
            YK_CUDA(cudaMemcpyAsync((char *)dst->ptr + dst_offset, (const char *)src->ptr + src_offset, bytes,
                                    cudaMemcpyDeviceToDevice, stream->s));
        record_completion(stream, completion);
    });
}

}  // extern "C"

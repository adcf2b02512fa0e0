// Host-side block allocator and block-table helpers of the paged KV pool: the
// counterpart of memory.Allocator / memory.Table (memory/memory.go:34-266), for
// hosts that keep the paging bookkeeping behind the C ABI. No device work here;
// the block ids it hands out are what yuuka_session_set_block_table takes.
#include <mutex>
#include <vector>

#include "common.cuh"

struct yuuka_allocator {
    int32_t block_size = 0;
    std::vector<int32_t> free;   // LIFO; filled descending so that the first acquire returns block 0 (memory.go:65-67)
    std::vector<int32_t> refs;
    uint64_t allocated = 0, released = 0;
    std::mutex mu;
};

using namespace yk;

extern "C" {

// NewAllocator, memory/memory.go:52-69
yuuka_status yuuka_allocator_create(int32_t blocks, int32_t block_size, yuuka_allocator ** out) {
    return guard([&] {
        YK_REQUIRE(out, YUUKA_ERR_INVALID_ARGUMENT, "allocator_create: null output");
        *out = nullptr;
        YK_REQUIRE(blocks > 0, YUUKA_ERR_INVALID_ARGUMENT, "memory: block count %d must be positive", blocks);
        YK_REQUIRE(block_size > 0, YUUKA_ERR_INVALID_ARGUMENT, "memory: block size %d must be positive", block_size);
        auto * a = new yuuka_allocator();
        a->block_size = block_size;
        a->refs.assign((size_t)blocks, 0);
        a->free.resize((size_t)blocks);
        for (int32_t i = 0; i < blocks; i++) a->free[(size_t)i] = blocks - 1 - i;
        *out = a;
    });
}

void yuuka_allocator_destroy(yuuka_allocator * a) { delete a; }

// Acquire, memory/memory.go:89-114 (without the evictor hook): YUUKA_ERR_ALLOCATION is ErrOutOfBlocks
yuuka_status yuuka_allocator_acquire(yuuka_allocator * a, int32_t * id) {
    return guard([&] {
        YK_REQUIRE(a && id, YUUKA_ERR_INVALID_ARGUMENT, "allocator_acquire: null argument");
        std::lock_guard<std::mutex> lock(a->mu);
        YK_REQUIRE(!a->free.empty(), YUUKA_ERR_ALLOCATION, "memory: out of blocks");
        *id = a->free.back();
        a->free.pop_back();
        a->refs[(size_t)*id] = 1;
        a->allocated++;
    });
}

// Retain, memory/memory.go:117-128
yuuka_status yuuka_allocator_retain(yuuka_allocator * a, int32_t id) {
    return guard([&] {
        YK_REQUIRE(a, YUUKA_ERR_INVALID_ARGUMENT, "allocator_retain: null allocator");
        std::lock_guard<std::mutex> lock(a->mu);
        YK_REQUIRE(id >= 0 && (size_t)id < a->refs.size(), YUUKA_ERR_INVALID_ARGUMENT, "memory: invalid block %d", id);
        YK_REQUIRE(a->refs[(size_t)id] > 0, YUUKA_ERR_INVALID_ARGUMENT, "memory: Retain of free block %d", id);
        a->refs[(size_t)id]++;
    });
}

// Release, memory/memory.go:132-147
yuuka_status yuuka_allocator_release(yuuka_allocator * a, int32_t id) {
    return guard([&] {
        YK_REQUIRE(a, YUUKA_ERR_INVALID_ARGUMENT, "allocator_release: null allocator");
        std::lock_guard<std::mutex> lock(a->mu);
        YK_REQUIRE(id >= 0 && (size_t)id < a->refs.size(), YUUKA_ERR_INVALID_ARGUMENT, "memory: invalid block %d", id);
        YK_REQUIRE(a->refs[(size_t)id] > 0, YUUKA_ERR_INVALID_ARGUMENT, "memory: Release of free block %d", id);
        a->released++;
        if (--a->refs[(size_t)id] == 0) a->free.push_back(id);
    });
}

// Refs, memory/memory.go:150-157: zero for an invalid block
int32_t yuuka_allocator_refs(yuuka_allocator * a, int32_t id) {
    if (!a) return 0;
    std::lock_guard<std::mutex> lock(a->mu);
    return id >= 0 && (size_t)id < a->refs.size() ? a->refs[(size_t)id] : 0;
}

// Stats, memory/memory.go:160-179
yuuka_status yuuka_allocator_stats_get(yuuka_allocator * a, yuuka_allocator_stats * out) {
    return guard([&] {
        YK_REQUIRE(a && out, YUUKA_ERR_INVALID_ARGUMENT, "allocator_stats_get: null argument");
        std::lock_guard<std::mutex> lock(a->mu);
        int32_t shared = 0;
        for (int32_t r : a->refs) shared += r > 1;
        out->block_size = a->block_size;
        out->total = (int32_t)a->refs.size();
        out->free = (int32_t)a->free.size();
        out->used = out->total - out->free;
        out->shared = shared;
        out->allocated = a->allocated;
        out->released = a->released;
    });
}

// Table.Cover / Table.Grow, memory/memory.go:203-233: grows blocks[0..*count) until it maps `positions`
// token positions; on failure the blocks acquired by this call are released and the table is unchanged.
yuuka_status yuuka_table_cover(yuuka_allocator * a, int32_t * blocks, int32_t * count, int32_t capacity, int32_t positions) {
    return guard([&] {
        YK_REQUIRE(a && blocks && count, YUUKA_ERR_INVALID_ARGUMENT, "table_cover: null argument");
        YK_REQUIRE(positions >= 0, YUUKA_ERR_INVALID_ARGUMENT, "memory: negative position coverage %d", positions);
        YK_REQUIRE(*count >= 0 && *count <= capacity, YUUKA_ERR_INVALID_ARGUMENT, "table_cover: invalid table length %d", *count);
        const int32_t need = (positions + a->block_size - 1) / a->block_size;
        YK_REQUIRE(need <= capacity, YUUKA_ERR_INVALID_ARGUMENT, "table_cover: %d blocks do not fit a table of %d", need, capacity);
        const int32_t start = *count;
        for (int32_t n = start; n < need; n++) {
            int32_t id = 0;
            if (yuuka_allocator_acquire(a, &id) != YUUKA_OK) {
                for (int32_t k = start; k < n; k++) yuuka_allocator_release(a, blocks[k]);
                throw StatusError{fail(YUUKA_ERR_ALLOCATION, "memory: out of blocks")};
            }
            blocks[n] = id;
        }
        if (need > start) *count = need;
    });
}

// Table.Map, memory/memory.go:256-266
yuuka_status yuuka_table_map(const int32_t * blocks, int32_t count, int32_t block_size, int32_t pos, int32_t * block,
                             int32_t * offset) {
    return guard([&] {
        YK_REQUIRE(blocks && block && offset && block_size > 0, YUUKA_ERR_INVALID_ARGUMENT, "table_map: invalid argument");
        YK_REQUIRE(pos >= 0, YUUKA_ERR_INVALID_ARGUMENT, "memory: negative position %d", pos);
        const int32_t index = pos / block_size;
        YK_REQUIRE(index < count, YUUKA_ERR_INVALID_ARGUMENT, "memory: position %d is not mapped by %d blocks", pos, count);
        *block = blocks[index];
        *offset = pos % block_size;
    });
}

}  // extern "C"

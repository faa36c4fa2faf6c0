// Symmetric heap (see symm_heap.cpp).
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>

namespace odc {

struct Heap;

Heap* heap_create(int rank, int world, int device, size_t bytes_per_rank, const std::string& mode,
                  const std::string& token);
// Collective: create `new_size - mapped` more bytes, exchange handles with every peer, map all.
void heap_grow(Heap* h, size_t new_size);
std::string heap_ipc_handle(Heap* h);
void heap_ipc_open(Heap* h, int rank, const std::string& handle);
uintptr_t heap_base(Heap* h, int rank);
size_t heap_mapped(Heap* h);
void heap_destroy(Heap* h);

std::string ipc_export(const void* device_ptr);
void* ipc_import(const std::string& blob);

}  // namespace odc

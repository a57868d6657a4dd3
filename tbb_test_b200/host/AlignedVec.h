// 64-byte aligned std::vector, the host staging container of the benchmark.
// Same public names as the reference's AlignedVec.h (aligned_allocator<T, A>,
// aligned_vector<T>; AlignedVec.h:14,122-123); written against the C++17 minimal
// allocator requirements.
#pragma once

#include <cstddef>
#include <cstdlib>
#include <limits>
#include <new>
#include <stdexcept>
#include <vector>

template <typename T, std::size_t Alignment>
class aligned_allocator {
 public:
  using value_type = T;
  using size_type = std::size_t;
  using difference_type = std::ptrdiff_t;
  template <typename U>
  struct rebind {
    using other = aligned_allocator<U, Alignment>;
  };

  aligned_allocator() noexcept = default;
  template <typename U>
  aligned_allocator(const aligned_allocator<U, Alignment>&) noexcept {}

  size_type max_size() const noexcept { return std::numeric_limits<size_type>::max() / sizeof(T); }

  T* allocate(size_type n) const {
    if (n == 0) return nullptr;
    if (n > max_size()) throw std::length_error("aligned_allocator: size overflow");
    // aligned_alloc wants a size that is a multiple of the alignment
    size_type bytes = (n * sizeof(T) + Alignment - 1) / Alignment * Alignment;
    void* p = std::aligned_alloc(Alignment, bytes);
    if (!p) throw std::bad_alloc();
    return static_cast<T*>(p);
  }
  void deallocate(T* p, size_type) const noexcept { std::free(p); }

  template <typename U>
  bool operator==(const aligned_allocator<U, Alignment>&) const noexcept { return true; }
  template <typename U>
  bool operator!=(const aligned_allocator<U, Alignment>&) const noexcept { return false; }
};

template <typename T>
using aligned_vector = std::vector<T, aligned_allocator<T, 64>>;

// Which layers' weight gradients are summed by one collective. Plain C++ (no CUDA) so that
// the host-side tests and the benchmark use the very rule the library applies.
#pragma once

#include <cstddef>

namespace b2 {

// Layers are visited in the order their gradients appear during backward (L-1 first) and
// closed into a bucket once the bucket holds `target` bytes:
//   ar_bucket_mb  > 0  target = that many MiB, every bucket the same;
//   ar_bucket_mb == 0, or nothing to sum (one rank / allreduce off): one layer per bucket;
//   ar_bucket_mb  < 0  (default) target = a quarter of all gradient bytes, at least 4 MiB, and
//                      with 4 or more ranks each later bucket 1.5 x the one before: there the
//                      chain of collectives outlasts the backward pass, so the first should
//                      start early and the rest be few; with 2 ranks the step is compute-bound
//                      and a small last bucket keeps the tail after the last gradient short.
// `growth` > 0 overrides the factor between consecutive buckets (values below 1 count as 1).
// Output per layer l: the lowest and highest layer index of its bucket.
inline void plan_gradient_buckets(const size_t* layer_bytes, int nlayers, int world_size, bool allreduce,
                                  int ar_bucket_mb, double growth, int* bucket_low, int* bucket_high) {
  size_t total = 0;
  for (int l = 0; l < nlayers; ++l) total += layer_bytes[l];
  const bool multi = world_size > 1 && allreduce;
  size_t target = total / 4;
  if (target < ((size_t)4 << 20)) target = (size_t)4 << 20;
  if (ar_bucket_mb == 0 || !multi) target = 0;
  if (ar_bucket_mb > 0) target = (size_t)ar_bucket_mb << 20;
  double factor = (ar_bucket_mb < 0 && world_size >= 4) ? 1.5 : 1.0;
  if (growth > 0.0) factor = growth;
  if (factor < 1.0) factor = 1.0;
  int high = nlayers - 1;
  size_t acc = 0;
  for (int l = nlayers - 1; l >= 0; --l) {
    acc += layer_bytes[l];
    if (acc >= target || l == 0) {
      for (int k = high; k >= l; --k) {
        bucket_low[k] = l;
        bucket_high[k] = high;
      }
      high = l - 1;
      acc = 0;
      target = (size_t)((double)target * factor);
    }
  }
}

// Sharded update (reduce-scatter, SGD on the owned slice, allgather): the step ends with the three
// of them for the bucket that holds layer 0, which nothing can overlap - its gradient is the last
// one produced and its weights are the first ones the next forward pass needs. Layer 0 therefore
// gets a bucket of its own (the rest of its former bucket stays together).
inline void plan_split_lowest_layer(int nlayers, int* bucket_low, int* bucket_high) {
  if (nlayers < 2 || bucket_high[0] == 0) return;
  const int high = bucket_high[0];
  for (int k = 1; k <= high; ++k) bucket_low[k] = 1;
  bucket_high[0] = 0;
}

// Layout of the gradient slab and of the weight slabs that mirror it: layers in the order
// backward produces their gradients (L-1 first), each padded to a multiple of 128 * world_size
// elements, so that every layer starts on a 256-byte boundary in a bf16 slab and every bucket
// of consecutive layers divides evenly among the ranks. Returns the slab's element count.
inline size_t plan_slab_layout(const size_t* layer_elems, int nlayers, int world_size, size_t* offset,
                               size_t* padded) {
  const size_t align = (size_t)128 * (size_t)(world_size < 1 ? 1 : world_size);
  size_t total = 0;
  for (int l = nlayers - 1; l >= 0; --l) {
    offset[l] = total;
    padded[l] = (layer_elems[l] + align - 1) / align * align;
    total += padded[l];
  }
  return total;
}

// Element range [begin, begin + count) of the bucket of layers [low, high] in the slabs, and
// the slice of it `rank` owns under the sharded update (the reduce-scatter leaves the sum of
// that slice with the rank, the rank updates those weights and the allgather distributes
// them): the reference's chunk ownership (mlp_omp.cc:80-94, 228) per bucket instead of per layer.
inline void plan_bucket_slice(const size_t* offset, const size_t* padded, int low, int high, int world_size, int rank,
                              size_t* begin, size_t* count, size_t* slice_begin, size_t* slice_count) {
  *begin = offset[high];
  *count = offset[low] + padded[low] - offset[high];
  const size_t per = *count / (size_t)world_size;
  if (slice_begin) *slice_begin = *begin + (size_t)rank * per;
  if (slice_count) *slice_count = per;
}

}  // namespace b2

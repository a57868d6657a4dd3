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

}  // namespace b2

#include "Rand.h"

#include <algorithm>
#include <cassert>
#include <numeric>
#include <random>
#include <vector>

#include "b2_rng.h"

namespace {
uint64_t g_seed = 3;  // the reference opens its quasi-random stream with dimension 3 (Rand.cc:20)
uint64_t g_pos = 0;
std::mt19937 g_int_engine(12345);

template <typename T>
void fill_ints(T* out, int len, int low, int high, bool duplicates) {
  if (duplicates) {
    std::uniform_int_distribution<T> pick(low, high);
    for (int i = 0; i < len; ++i) out[i] = pick(g_int_engine);
    return;
  }
  // distinct values: partial Fisher-Yates over [low, high]
  const int64_t span = (int64_t)high - low + 1;
  assert(span >= len);
  std::vector<T> pool((size_t)span);
  std::iota(pool.begin(), pool.end(), (T)low);
  for (int i = 0; i < len; ++i) {
    std::uniform_int_distribution<int64_t> pick(i, span - 1);
    std::swap(pool[(size_t)i], pool[(size_t)pick(g_int_engine)]);
    out[i] = pool[(size_t)i];
  }
}
}  // namespace

void randSeed(uint64_t seed, uint64_t position) {
  g_seed = seed;
  g_pos = position;
}

void randFill(float* array, size_t len, const float low, const float high, bool) {
  for (size_t i = 0; i < len; ++i) array[i] = b2_rng_uniform(g_seed, g_pos + i, low, high);
  g_pos += len;
}

void randFill(double* array, size_t len, const double low, const double high, bool) {
  for (size_t i = 0; i < len; ++i) array[i] = (double)b2_rng_uniform(g_seed, g_pos + i, (float)low, (float)high);
  g_pos += len;
}

void randFill(int* array, int len, const int low, const int high, bool duplicates) {
  fill_ints(array, len, low, high, duplicates);
}
void randFill(int64_t* array, int len, const int low, const int high, bool duplicates) {
  fill_ints(array, len, low, high, duplicates);
}
void randFill(aligned_vector<float>& vec, const float low, const float high) {
  randFill(vec.data(), vec.size(), low, high);
}
void randFill(aligned_vector<double>& vec, const double low, const double high) {
  randFill(vec.data(), vec.size(), low, high);
}
void randFill(aligned_vector<int>& vec, const int low, const int high, bool duplicates) {
  randFill(vec.data(), (int)vec.size(), low, high, duplicates);
}
void randFill(aligned_vector<int64_t>& vec, const int low, const int high, bool duplicates) {
  randFill(vec.data(), (int)vec.size(), low, high, duplicates);
}

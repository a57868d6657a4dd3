// Uniform fills for the benchmark's matrices: same overload set as the reference's
// Rand.h:7-28.  Floating-point fills draw from the portable counter-based stream of
// include/b2_rng.h (the reference's MKL Niederreiter stream, Rand.cc:14-49, cannot be
// reproduced without MKL), consumed sequentially from a process-wide position that
// randSeed() rewinds; integer fills use std::mt19937.
#pragma once

#include <cstddef>
#include <cstdint>

#include "AlignedVec.h"

void randSeed(uint64_t seed, uint64_t position = 0);

void randFill(aligned_vector<float>& vec, const float low, const float high);
void randFill(aligned_vector<double>& vec, const double low, const double high);
void randFill(aligned_vector<int>& vec, const int low, const int high, bool duplicates = true);
void randFill(aligned_vector<int64_t>& vec, const int low, const int high, bool duplicates = true);
void randFill(float* array, size_t len, const float low, const float high, bool duplicates = true);
void randFill(double* array, size_t len, const double low, const double high, bool duplicates = true);
void randFill(int* array, int len, const int low, const int high, bool duplicates = true);
void randFill(int64_t* array, int len, const int low, const int high, bool duplicates = true);

// Host matrix of the benchmark: row-major, leading dimension ncols + PAD,
// (nrows + PAD) * (ncols + PAD) elements, 4 KiB aligned.  Same public surface as
// the reference's Matrix<T, PAD> (Matrix.h:18-203) so that driver code written
// against it compiles unchanged; the device library reads and writes these
// buffers through (pointer, ld) pairs and never takes ownership.
//
// Ownership follows the reference: a Matrix frees its pointer on destruction,
// including one adopted through the wrapping constructor or assign()
// (Matrix.h:20-22,35-40,133-138) - never hand it device or pinned memory.
#ifndef B2_HOST_MATRIX_H
#define B2_HOST_MATRIX_H

#include <algorithm>
#include <cassert>
#include <cmath>
#include <cstdlib>
#include <iomanip>
#include <iostream>
#include <string>
#include <vector>

#include "Rand.h"

template <typename T, int PAD = 0>
class Matrix {
 public:
  Matrix(const int nrows, const int ncols, const std::string name = "")
      : data_(nullptr), nrows_(nrows), ncols_(ncols), name_(name) {
    check_shape();
    allocate();
  }

  Matrix(const int nrows, const int ncols, T* ptr, const std::string name = "")
      : data_(ptr), nrows_(nrows), ncols_(ncols), name_(name) {
    check_shape();
  }

  explicit Matrix(const std::vector<int> shape, const T low = T(0), const T high = T(0),
                  bool duplicates = true, const std::string name = "")
      : data_(nullptr), nrows_(shape.at(0)), ncols_(shape.at(1)), name_(name) {
    assert(shape.size() == 2);
    check_shape();
    allocate();
    for (int r = 0; r < nrows_; ++r) std::fill_n(rawData(r, 0), ncols_, low);
    if (low < high) randFill(low, high, duplicates);
  }

  Matrix(const Matrix&) = delete;
  Matrix& operator=(const Matrix&) = delete;
  ~Matrix() { std::free(data_); }

  void newInput(const T low = T(0), const T high = T(0), bool duplicates = true) {
    if (low < high) {
      randFill(low, high, duplicates);
    } else {
      std::fill(data_, data_ + padded_elems(), T(0));
    }
  }

  T& operator()(int row, int col) { return data_[offset(row, col)]; }
  const T& operator()(int row, int col) const { return data_[offset(row, col)]; }

  T* rawData() { return data_; }
  const T* rawData() const { return data_; }
  T* rawData(int row, int col) { return data_ + (size_t)row * ld() + col; }
  const T* rawData(int row, int col) const { return data_ + (size_t)row * ld() + col; }

  size_t size() const { return (size_t)nrows_ * ncols_; }

  void realloc(int nrows, int ncols) {
    std::free(data_);
    data_ = nullptr;
    nrows_ = nrows;
    ncols_ = ncols;
    check_shape();
    allocate();
  }
  void realloc(const std::vector<int>& shape) { realloc(shape.at(0), shape.at(1)); }

  // Adopts the vector's storage as a dense nrows x ncols block (ld() still reports
  // ncols + PAD, as in the reference).
  void assign(aligned_vector<T>& other, int nrows, int ncols) {
    assert((size_t)nrows * ncols == other.size());
    nrows_ = nrows;
    ncols_ = ncols;
    data_ = other.data();
  }

  std::vector<int> shape() const { return {nrows_, ncols_}; }
  std::string name() const { return name_; }
  int nrows() const { return nrows_; }
  int ncols() const { return ncols_; }
  int ld() const { return ncols_ + PAD; }

  // Element-wise comparison over the first size() elements of the buffer with a
  // relative tolerance of 1e-6 (Matrix.h:150-162).
  bool operator==(const Matrix& other) const {
    const double rtol = 1e-6;
    for (size_t i = 0; i < size(); ++i) {
      const double a = rawData()[i], b = other.rawData()[i];
      if (std::abs(a - b) > rtol * std::abs(b)) {
        std::cout << rawData()[i] << " " << other.rawData()[i] << "\n";
        return false;
      }
    }
    return true;
  }

  void randFill(T low, T high, bool duplicates = true) {
    for (int r = 0; r < nrows_; ++r) ::randFill(rawData(r, 0), (size_t)ncols_, low, high, duplicates);
  }

  T* data_;

 protected:
  size_t padded_elems() const { return ((size_t)nrows_ + PAD) * ((size_t)ncols_ + PAD); }
  size_t offset(int row, int col) const {
    assert(row >= 0 && row < nrows_ && col >= 0 && col < ncols_);
    return (size_t)row * ld() + col;
  }
  void check_shape() const {
    assert(nrows_ > 0);
    assert(ncols_ > 0);
  }
  void allocate() {
    void* p = nullptr;
    if (posix_memalign(&p, 4096, sizeof(T) * padded_elems()) != 0) p = nullptr;
    data_ = static_cast<T*>(p);
    assert(data_);
  }

  int nrows_;
  int ncols_;
  std::string name_;
};

#define Const(x) (x)
#define From(x) (x)
#define To(x) (x)

inline std::vector<int> shape(int nrows, int ncols) { return {nrows, ncols}; }

template <typename T>
T sum(Matrix<T>& m) {
  T total = T(0);
  for (size_t i = 0; i < m.size(); ++i) total += m.rawData()[i];
  return total;
}

template <typename T, int PAD>
std::ostream& operator<<(std::ostream& os, const Matrix<T, PAD>& m) {
  os << "Matrix " << m.name() << ": " << m.nrows() << " x " << m.ncols() << "\n";
  for (int r = 0; r < m.nrows(); ++r) {
    for (int c = 0; c < m.ncols(); ++c) os << std::setprecision(9) << m(r, c) << " ";
    os << "\n";
  }
  return os;
}

#endif

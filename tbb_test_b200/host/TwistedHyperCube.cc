#include "TwistedHyperCube.h"

#include <cassert>

HyperCube::HyperCube(int num_nodes, int shift) : num_nodes_(num_nodes), shift_(shift) {}

int HyperCube::NumNodes() const { return num_nodes_; }

int HyperCube::Dimension() const {
  int dim = 0;
  while ((1 << dim) < num_nodes_) ++dim;
  assert((1 << dim) == num_nodes_);
  return dim;
}

// Rotate the low Dimension() bits of `id` left by `shift`.
int HyperCube::ShiftedId(int id, int shift) const {
  const int d = Dimension();
  const int mask = (1 << d) - 1;
  return ((id << shift) | (id >> (d - shift))) & mask;
}

int HyperCube::ShiftedId(int id) const { return ShiftedId(id, shift_); }

int HyperCube::UnshiftedId(int id) const { return ShiftedId(id, Dimension() - shift_); }

int HyperCube::Peer(int id, int dim) const {
  assert(id >= 0 && id < num_nodes_);
  return UnshiftedId(ShiftedId(id) ^ (1 << dim));
}

int HyperCube::RecvLocation(int id, int dim) const {
  assert(dim >= 0 && dim < Dimension());
  // bit `dim` of the rotated id picks the half kept in this step; higher dimensions
  // (earlier steps) have already fixed the enclosing range
  int location = 0;
  const int sid = ShiftedId(id);
  for (int d = dim; d < Dimension(); ++d) location += sid & (1 << d);
  return location;
}

int HyperCube::SendLocation(int id, int dim) const { return RecvLocation(Peer(id, dim), dim); }

TwistedHyperCube::TwistedHyperCube(int num_nodes, int shift) : HyperCube(num_nodes, shift) {
  assert(num_nodes <= 8);
}

int TwistedHyperCube::Peer(int id, int dim) const {
  const int d = Dimension();
  const int link = (dim - shift_ + d) % d;
  // link k flips the k+1 lowest bits; the two cross links of the twist (2-5, 3-4 in
  // plain numbering) are rewired to 2-4 and 3-5
  const int plain = id ^ ((1 << (link + 1)) - 1);
  if (id == 2 && plain == 5) return 4;
  if (id == 3 && plain == 4) return 5;
  if (id == 4 && plain == 3) return 2;
  if (id == 5 && plain == 2) return 3;
  return plain;
}

int TwistedHyperCube::RecvLocation(int id, int dim) const {
  const int d = Dimension();
  assert(dim >= 0 && dim < d);
  int location = 0;
  for (int step = dim; step < d; ++step) {
    const int link = (step - shift_ + d) % d;
    int offset = 0;
    if (num_nodes_ == 8 && shift_ > 0 && step >= 1) {
      // rotated 8-node case: the halves are fixed by tables (TwistedHyperCube.cc:91-103)
      if (step == 2) {
        offset = (id >= 2 && id <= 5) ? 4 : 0;
      } else {
        offset = (id == 1 || id == 2 || id == 4 || id == 6) ? 2 : 0;
      }
    } else if (link == 0) {
      // the lowest link pairs 0-1 and 3-2 inside each square
      const int low2 = id & 3;
      offset = (low2 == 1 || low2 == 2) ? (1 << shift_) : 0;
    } else if (link + shift_ >= d) {
      offset = (id & (1 << link)) >> (d - shift_);
    } else {
      offset = (id & (1 << link)) << shift_;
    }
    location += offset;
  }
  return location;
}

int TwistedHyperCube::SendLocation(int id, int dim) const { return RecvLocation(Peer(id, dim), dim); }

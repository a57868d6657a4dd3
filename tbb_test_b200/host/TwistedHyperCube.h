// Peer and chunk addressing for recursive halving / doubling on a hypercube and on
// the 8-socket "twisted" hypercube (two squares 0-1-2-3 and 4-5-6-7 whose cross
// links are 0-7, 1-6, 2-4, 3-5).  Same classes and methods as the reference's
// TwistedHyperCube.h:3-48.
//
// In step `dim` of a recursive-halving reduce-scatter node `id` exchanges with
// Peer(id, dim); it keeps (receives into) the half of its current chunk range that
// starts at chunk RecvLocation(id, dim) and sends the half that starts at
// SendLocation(id, dim). Recursive doubling (allgather) walks the dimensions in the
// opposite order: pass Dimension() - 1 - dim.
#pragma once

class HyperCube {
 public:
  // `shift` rotates the bits of the node id, i.e. which physical link serves
  // which dimension.
  HyperCube(int num_nodes, int shift = 0);
  virtual ~HyperCube() = default;

  int NumNodes() const;
  int Dimension() const;
  virtual int Peer(int id, int dim) const;
  virtual int RecvLocation(int id, int dim) const;
  virtual int SendLocation(int id, int dim) const;

 protected:
  int ShiftedId(int id, int shift) const;
  int ShiftedId(int id) const;
  int UnshiftedId(int id) const;

  int num_nodes_;
  int shift_;
};

class TwistedHyperCube : public HyperCube {
 public:
  TwistedHyperCube(int num_nodes, int shift = 0);

  int Peer(int id, int dim) const override;
  int RecvLocation(int id, int dim) const override;
  int SendLocation(int id, int dim) const override;
};

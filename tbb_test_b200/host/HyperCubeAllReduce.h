// A data path for the HyperCube / TwistedHyperCube addressing (the reference declares the
// classes, TwistedHyperCube.h:3-48, but never moves data with them): recursive-halving
// reduce-scatter followed by recursive-doubling allgather over `NumNodes()` equal-length
// buffers, one per node, all in this process' memory.
//
// The buffers are cut into NumNodes() chunks (chunk c = elements [c*chunk, (c+1)*chunk),
// the last one shorter when the length does not divide). Halving walks the dimensions from
// the highest to 0: in dimension d node i adds, into the 2^d chunks starting at
// RecvLocation(i, d), the same chunks of Peer(i, d) - which that peer gives up
// (SendLocation(peer, d) == RecvLocation(i, d)). After dimension 0 node i holds the full sum
// of chunk RecvLocation(i, 0). Doubling walks the dimensions upwards and copies the
// peer's finished chunks back. Steps are separated by a barrier between all nodes, so the
// result (and the order of every floating-point sum) does not depend on thread timing.
//
// HyperCubeStep lists what one node does in one step; a device implementation executes the
// same list with peer loads over NVLink.
#pragma once

#include <cstddef>
#include <vector>

#include "TwistedHyperCube.h"

struct HyperCubeStep {
  int dim;         // dimension whose link is used
  int peer;        // node exchanged with
  int first_chunk; // first chunk this node reads from the peer
  int num_chunks;  // 2^dim
  bool reduce;     // true: add the peer's chunks into mine (halving); false: copy them (doubling)
};

// The 2 * Dimension() steps of node `id`: halving then doubling.
std::vector<HyperCubeStep> hypercube_allreduce_steps(const HyperCube& cube, int id);

// True when the addressing is usable as an allreduce schedule: every dimension pairs the
// nodes up, partners agree on the chunks they exchange, and the chunks owned after halving
// are a permutation. (False for the 8-node twisted cube with shift 2, whose special case in
// the reference is written for shift 1 only.)
bool hypercube_schedule_is_consistent(const HyperCube& cube);

// In-place sum of bufs[0..N) (each `count` floats) into every buffer. One thread per node
// when `threaded`, otherwise the nodes are walked step by step on the calling thread.
// `iterations` > 1 repeats the allreduce on its own result (for timing: the node threads are
// started once). Returns false (buffers untouched) when the schedule is inconsistent.
bool hypercube_allreduce(const HyperCube& cube, float* const* bufs, size_t count, bool threaded,
                         int iterations = 1);

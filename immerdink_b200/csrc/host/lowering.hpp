// Index-map lowering: labelled strided tensors -> batched GEMM view. CUDA-free.
//
// Behaviour follows the reference's lowering (src/host/index_map.cpp:93-239; normative text
// docs/DESIGN.md:1526-1597): label classes I {A,C}, J {B,C}, K {A,B}/{A}/{B}, L {A,B,C};
// legality rows in precedence order; the role swap that makes the GEMM's column index run
// along C's fastest mode; canonical mode orders; fusion of modes that are contiguous in every
// tensor.
#pragma once
#include <cstdint>
#include <vector>

#include "immerdink/immerdink_host.h"

namespace imd {

enum : int { kClsI = 0, kClsJ = 1, kClsK = 2, kClsL = 3 };
enum : int { kTenA = 0, kTenB = 1, kTenC = 2 };

struct Label {
  int32_t id = 0;
  int64_t extent = 0;
  int first = 0;                 // first position in A.labels ++ B.labels ++ C.labels
  int count[3] = {0, 0, 0};      // occurrences per tensor (post-swap frame after lowering)
  int64_t stride[3] = {0, 0, 0}; // merged (diagonal) stride per tensor, post-swap frame
  int cls = kClsK;
};

struct Mode {                    // a fused run of labels of one class
  int64_t extent = 1;
  int64_t stride[3] = {0, 0, 0};
};

struct GemmView {
  int64_t m = 0, n = 0, k = 0, b = 0;  // post-swap sizes of I, J, K, L
  bool swapped = false;
  std::vector<Label> labels;
  std::vector<int32_t> order[4];       // canonical label order per class, first = fastest
  std::vector<Mode> modes[4];          // fused modes per class, first = fastest
  bool empty_output() const { return b == 0 || m == 0 || n == 0; }
  int64_t vec_entries() const { return 2 * m + 2 * n + 2 * k + 3 * b; }
};

imd_status_t lower(const imd_tensor_t& A, const imd_tensor_t& B, const imd_tensor_t& C,
                   GemmView* out);

const Label* find_label(const GemmView& v, int32_t id);
// Replace the canonical order of class `cls` (a permutation of its kept labels) and redo the fusion.
void adopt_order(GemmView* v, int cls, const std::vector<int32_t>& order);

// Offsets of tensor X over the fused modes of class `cls` (mixed radix, first mode fastest).
void scatter_vector(const GemmView& v, int cls, int X, int64_t* out);
// The nine vectors in region order: A row, k, batch; B k, col, batch; C row, col, batch.
void scatter_vectors(const GemmView& v, int64_t* out);

}  // namespace imd

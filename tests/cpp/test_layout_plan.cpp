// Unit test of the strided-copy planner (tensorvia_b200/csrc/layout_plan.h): which kernel a
// view gets and how its indices merge.  Host only.
#include <cstdio>
#include <cstdlib>

#include "layout_plan.h"

using namespace tvb;

#define CHECK(cond)                                                        \
  do {                                                                     \
    if (!(cond)) {                                                         \
      std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);        \
      std::exit(1);                                                        \
    }                                                                      \
  } while (0)

int main() {
  {  // a dense tensor is one run whatever its rank
    LayoutDim d[3] = {{4, 30, 30}, {5, 6, 6}, {6, 1, 1}};
    CopyPlan p = plan_copy(d, 3, 4, 0, 0);
    CHECK(p.kind == CopyKind::kContiguous && p.ndim == 1 && p.dim[0].size == 120);
  }
  {  // a window of leading rows too
    LayoutDim d[2] = {{3, 8, 8}, {8, 1, 1}};
    CHECK(plan_copy(d, 2, 2, 0, 0).kind == CopyKind::kContiguous);
  }
  {  // inner window: rows of 6 floats out of 8, 8-byte vectors (6*4 = 24 is not a multiple of 16)
    LayoutDim d[2] = {{5, 8, 6}, {6, 1, 1}};
    CopyPlan p = plan_copy(d, 2, 4, 0, 0);
    CHECK(p.kind == CopyKind::kVector && p.ndim == 2 && p.vector_bytes == 8);
    // a base that is only 4-byte aligned narrows the vector
    CHECK(plan_copy(d, 2, 4, 4, 0).vector_bytes == 4);
    // rows of 8 halves in a pitch of 16: 16-byte vectors
    LayoutDim h[2] = {{5, 16, 8}, {8, 1, 1}};
    CHECK(plan_copy(h, 2, 2, 0, 0).vector_bytes == 16);
    // an odd pitch of bytes: single bytes
    LayoutDim b[2] = {{5, 7, 3}, {3, 1, 1}};
    CHECK(plan_copy(b, 2, 1, 0, 0).vector_bytes == 1);
  }
  {  // t() of a [7,5] array: the source is contiguous along the outer index
    LayoutDim d[2] = {{5, 1, 7}, {7, 5, 1}};
    CopyPlan p = plan_copy(d, 2, 4, 0, 0);
    CHECK(p.kind == CopyKind::kTranspose && p.unit_dim == 0 && p.ndim == 2);
  }
  {  // permute {0,2,1} of [3,4,5]: batch outermost, then the transposed plane
    LayoutDim d[3] = {{3, 20, 20}, {5, 1, 4}, {4, 5, 1}};
    CopyPlan p = plan_copy(d, 3, 2, 0, 0);
    CHECK(p.kind == CopyKind::kTranspose && p.unit_dim == 1 && p.ndim == 3);
  }
  {  // permute {1,0,2} of [3,4,5]: innermost runs stay contiguous -> vector copy of rows
    LayoutDim d[3] = {{4, 5, 15}, {3, 20, 5}, {5, 1, 1}};
    CopyPlan p = plan_copy(d, 3, 4, 0, 0);
    CHECK(p.kind == CopyKind::kVector && p.ndim == 3 && p.vector_bytes == 4);
  }
  {  // no contiguous run in the source at all
    LayoutDim d[2] = {{4, 10, 3}, {3, 2, 1}};
    CHECK(plan_copy(d, 2, 4, 0, 0).kind == CopyKind::kElement);
  }
  {  // extents of 1 vanish; a single element is a contiguous copy of one
    LayoutDim d[3] = {{1, 99, 1}, {1, 7, 1}, {1, 3, 1}};
    CopyPlan p = plan_copy(d, 3, 8, 0, 0);
    CHECK(p.kind == CopyKind::kContiguous && p.dim[0].size == 1);
    LayoutDim e[3] = {{1, 99, 12}, {4, 1, 3}, {3, 4, 1}};
    CopyPlan q = plan_copy(e, 3, 4, 0, 0);
    CHECK(q.kind == CopyKind::kTranspose && q.ndim == 2 && q.unit_dim == 0);
  }
  {  // a concat part: `outer` dense runs landing further apart
    LayoutDim d[2] = {{6, 12, 40}, {12, 1, 1}};
    CopyPlan p = plan_copy(d, 2, 2, 0, 0);
    CHECK(p.kind == CopyKind::kVector && p.vector_bytes == 8);
    LayoutDim one[2] = {{1, 12, 40}, {12, 1, 1}};
    CHECK(plan_copy(one, 2, 2, 0, 0).kind == CopyKind::kContiguous);
  }
  std::printf("all checks passed\n");
  return 0;
}

// C wrapper around the reference's CpBalanceSolver header (included from the
// reference checkout at build time, never copied): the checker's exact IPO
// partition oracle.
#include "cp_balance_fast.hpp"

extern "C" int ref_ipo_solve(const int* weights, int n, int m, int* assign_out) {
  return CpBalanceSolver::solve_to(weights, n, m, assign_out);
}

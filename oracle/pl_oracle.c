/* TEST INFRASTRUCTURE ONLY: the checker for the CUDA path and the timed CPU baseline.
 * Nothing in the product may call into this file.
 *
 * CPU restatement, in plain C, of the reference's fp32 CPU lattice filter
 * (src/PermutohedralLatticeCPU.h of MiguelMonteiro/permutohedral_lattice, T = float), written so
 * that every floating-point operation happens in the same precision and order as in that header
 * compiled with g++ -O2 -ffp-contract=off.  Build this file with -ffp-contract=off too.
 *
 * Parity status: PINNED.  tests/test_oracle_vs_reference.py checks it bit-for-bit (outputs, vertex
 * keys in creation order, per-pixel vertex ids and weights) against the unmodified header
 * (oracle/ref_shim.cpp) wherever the reference tree is present, and tests/test_oracle_golden.py
 * checks it against fixtures under tests/golden/ that were produced by that header.
 *
 * The same code is instantiated for T = double (plo_*_f64 entry points), including the reference's quirk
 * of keeping one product of the elevation step in a float (src/PermutohedralLatticeCPU.h:226).
 *
 * One deliberate difference: the reference's hash table keeps probing from a stale bucket after it
 * grows (src/PermutohedralLatticeCPU.h:59-62,163-165) and so creates duplicate vertices.  The table
 * here rehashes correctly, which equals the reference run with a table large enough never to grow.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#define PLO_CAT2(a, b) a##b
#define PLO_CAT(a, b) PLO_CAT2(a, b)

#define REAL float
#define N(name) name
#include "pl_oracle_impl.h"
#undef REAL
#undef N

#define REAL double
#define N(name) PLO_CAT(name, _f64)
#include "pl_oracle_impl.h"
#undef REAL
#undef N

// Internal declarations shared by the host inspector, the planner and the CUDA side.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "tile_fusion_b200.h"

struct tf_schedule {
  int n1 = 0;
  std::vector<int> ptr1, ptr2, id, type, ker;  // ker empty = absent
  bool has_ker = false;
  double stats[5] = {0, 0, 0, 0, 0};
};

namespace tf {

constexpr int kDefaultTileSlots = 800;  // 100 KB of staging per CTA: two CTAs per SM
constexpr int kDefaultTileSlotsSmall = kDefaultTileSlots;
// tile pipeline: 3 x 512 x 128 B of chunk buffers + 2 x 8 x 256 x 8 B of row tables = 229 376 B per SM
constexpr int kPipeTileSlots = 512;
constexpr int kPipeTileRows = 256;
constexpr int kDefaultTileMaxBz = 8;
constexpr int kHeavyRowNnz = 256;    // a row at least this long is a block of its own (the CTA's warps share it)
constexpr int kSegmentNnz = 4096;    // a row longer than this is cut into segments run by different CTAs
constexpr bool kDefaultTileDoubleBuffer = false;
constexpr int kTileMaxRows = 512;        // rows of a gather tile (16 per 8-lane group of a 256-thread CTA)

void set_error(const std::string &msg);
int fail(int code, const std::string &msg);

// Work item of the persistent executor (two int4 on the device).
enum ItemKind : int {
  ITEM_PRODUCE = 0, ITEM_CONSUME = 1, ITEM_SDDMM = 2, ITEM_SEND = 3,
  ITEM_PRODUCE_TILED = 4,  // row_begin = tile index of the first operator's tiling
  ITEM_CONSUME_TILED = 5,  // row_begin = tile index of the second operator's tiling
  // heavy-row segments: row_begin = row, row_end = first nonzero, base = one past the last nonzero
  ITEM_PRODUCE_SEG = 6, ITEM_CONSUME_SEG = 7, ITEM_SDDMM_SEG = 8
};
struct Item {
  int kind;       // ItemKind
  int block;      // index into the producer / consumer done-flag array
  int row_begin;  // first row of the block
  int row_end;    // one past the last row
  int need;       // watermark of the other side this item waits for
  int base;       // consumer: ring origin of its column window (multiple of ring_rows)
  int aux0, aux1;
};

// Lattice structure of a pattern: the dominant column offsets are 1, nx and nx*ny around the operator's
// own diagonal, which sits `shift` columns right of the row index (0 for a square operator; a constant
// when the columns were renumbered, as for one rank's rows of a partitioned chain).
struct Lattice {
  int dims = 0;  // 0 = none
  int nx = 0, ny = 0;
  int shift = 0;
};
Lattice detect_lattice(int m, const int *ap, const int *ai);

// An operator verified to be a star stencil (at most the 7 points 0, +-1, +-nx, +-nx*ny, never across a
// grid edge) on an nx x ny x nz lattice in natural order, with its rows classified by coefficient vector
// (see lattice.cpp).  This is what the plane-marching executor runs from instead of the CSR arrays.
constexpr int kMarchMaxClasses = 63;
struct LatticeOp {
  bool ok = false;
  int nx = 0, ny = 0, nz = 0;
  int ghost_lo = 0, ghost_hi = 0;  // planes of the source operand below / above the operator's own rows
  int n_classes = 0;               // distinct coefficient vectors; class n_classes is the all-zero vector
  std::vector<float> dict;         // (n_classes + 1) x 8: {z-, y-, x-, centre, x+, y+, z+, 0} -- CSR order
  std::vector<uint32_t> patch_cls; // [nz][ceil(ny/2)][ceil(nx/2)]: classes of the rows (2px+dx, 2py+dy, z), byte 2*dy+dx
};
// halo_lo / halo_hi: rows of source planes that are not addressed as shifted lattice neighbours but are
// appended after the m local rows (the second operator of a partitioned chain): lower plane first.
int analyse_lattice_operator(int m, int ncols, const int *ap, const int *ai, const float *ax, int halo_rows,
                             LatticeOp &out);

// Work items of the plane-marching executor: an x-y tile, a range of planes and a column chunk each.
struct MarchItem {
  int x0, y0, zs, ze, c0, flags;
};
// tile_w x tile_h tiles, chunks of `chunk` columns; planes [z_begin, z_end) cut into the number of segments
// that finishes soonest on `ctas` resident CTAs.  Order: segment, tile, chunk (chunks of a tile adjacent, so
// that concurrently running CTAs read whole dense rows and neighbouring tiles together).
void build_march_items(int nx, int ny, int z_begin, int z_end, int n_cols, int tile_w, int tile_h, int chunk,
                       int ctas, int min_segments, std::vector<MarchItem> &out);

// Partition of an operator's rows into gather tiles (see tiling.cpp).
struct Tiling {
  bool tiled = false, failed = false;
  int nx = 0, ny = 0, bx = 0, by = 0, bz = 0;
  std::vector<int> tile_row_ptr, rows;    // tile -> its output rows
  std::vector<int> tile_halo_ptr, halo;   // tile -> the source rows it stages, in slot order
  std::vector<uint16_t> slot;             // per nonzero of the operator: slot of its column in the tile
  double reuse = 0;                       // nonzeros per staged row
  int tiles() const { return tile_row_ptr.empty() ? 0 : (int)tile_row_ptr.size() - 1; }
};
int build_tiling(int m, const int *ap, const int *ai, int slot_cap, int max_bz, int max_rows, Tiling &out);

// A unit of the direct (untiled) path: rows [r0, r1), or -- for a row too heavy for one CTA -- the
// nonzeros [p0, p1) of the single row r0 (seg), whose partial sums are added atomically.
struct Unit {
  int r0, r1, p0, p1;
  bool seg;
};

// Host-side execution plan (what the planner derives from the patterns).
struct HostPlan {
  std::vector<Unit> prod_units;  // producer row blocks / heavy-row segments; empty when tiled
  std::vector<Unit> cons_units;  // consumer row blocks / heavy-row segments; empty when tiled
  std::vector<int> seg_t_rows;   // rows of T accumulated from segments (zeroed before a pass)
  std::vector<int> seg_out_rows; // rows of D accumulated from segments (zeroed before, ReLU after)
  int n_prod = 0, n_cons = 0;  // units (blocks or tiles) on each side
  std::vector<Item> items;     // all items in ticket order
  int phase_begin[4] = {0, 0, 0, 0};  // item ranges of the three phases
  long long ring_rows = 0;     // 0 = intermediate holds every row
  long long inter_rows = 0;    // rows allocated for the intermediate
};

struct PlanParams {
  int m = 0;             // local rows
  int n_cols = 0;        // dense width of the intermediate
  int rows_per_block = 0;
  long long ring_bytes = 0;
  int slack_blocks = -1;
  int max_ctas = 0;      // CTAs that will be resident (for the default slack)
  bool producer_is_gemm = false;
  int halo_rows = 0;
  std::vector<int> boundary_rows;
  int max_block_nnz = 0;
};

// first: CSR pattern of the first operator (nullptr for a dense producer); second: of A.
int build_stream_plan(const PlanParams &pp, const int *first_ap, const int *first_ai, const int *sec_ap,
                      const int *sec_ai, const Tiling *ptile, const Tiling *ctile, HostPlan &out);
int build_single_pass_plan(const PlanParams &pp, const int *ap, HostPlan &out);

int check_csr(int m, int ncols, const int *ap, const int *ai, bool need_sorted);

// Row-block partition of a chain over ranks (multi.cu): what one rank exchanges with the others.
struct ExchangeSegment {
  int peer;
  long long start, count;        // rows inside the halo buffer (receive) or the send buffer (send)
  std::vector<long long> index;  // send side: rows of the send buffer to gather when they are not consecutive
};
struct RankLayout {
  std::vector<long long> halo_ids;       // sorted global ids of the rows of T received
  std::vector<long long> boundary_rows;  // sorted LOCAL ids of the rows of T sent
  std::vector<ExchangeSegment> recv, send;
};
std::vector<long long> halo_of(const long long *ai, long long nnz, long long r0, long long r1);
int make_layout(int rank, int world, const long long *bounds, const std::vector<std::vector<long long>> &halos,
                RankLayout &out);

}  // namespace tf

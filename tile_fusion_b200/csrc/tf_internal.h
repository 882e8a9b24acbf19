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

}  // namespace tf

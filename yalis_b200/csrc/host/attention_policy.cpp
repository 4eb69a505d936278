// Launch model of the prompt-attention kernel (host only, no CUDA): how a step's tiles of queries should share
// their keys among blocks.  It runs once per step on the path that launches kernels, so it is native: the same
// model in Python took 2 to 5 ms for a step of 64 decoding requests beside a 512-token portion.
//
// A step is a list of items (key tiles, pace), one per tile of queries of one KV head.  With `splits` shares an
// item of more than `limit` key tiles is cut into ceil(tiles / limit) shares (at most `splits`); every share is
// a block that costs its key tiles times the item's pace plus a start-up.  Blocks run in launch order (share
// after share, items in order within a share), each on the first of `slots` places to come free; the step's
// length is when the last one ends.

#include <algorithm>
#include <cstdint>
#include <functional>
#include <queue>
#include <vector>

#define YPOL_API extern "C" __attribute__((visibility("default")))

namespace {

double step_length(const int32_t* tiles, const double* pace, int n_items, int slots, int splits, int limit,
                   double start_up) {
  std::priority_queue<double, std::vector<double>, std::greater<double>> free_at;
  for (int i = 0; i < slots; ++i) free_at.push(0.0);
  double end = 0.0;
  for (int z = 0; z < splits; ++z) {
    for (int i = 0; i < n_items; ++i) {
      const int t = tiles[i];
      const int wanted = splits > 1 ? std::min(splits, (t + limit - 1) / limit) : 1;
      const int per_share = (t + wanted - 1) / wanted;
      if ((long long)z * per_share >= t) continue;
      const int mine = std::min(t, (z + 1) * per_share) - z * per_share;
      const double done = free_at.top() + mine * pace[i] + start_up;
      free_at.pop();
      free_at.push(done);
      end = std::max(end, done);
    }
  }
  return end;
}

}  // namespace

YPOL_API double ypol_step_length(const int32_t* tiles, const double* pace, int n_items, int slots, int splits,
                                 int limit, double start_up) {
  if (n_items <= 0 || slots <= 0 || splits <= 0 || limit <= 0) return 0.0;
  return step_length(tiles, pace, n_items, slots, splits, limit, start_up);
}

// (kv_splits, tiles_per_split) for a step whose request i brings q_lens[i] tokens behind before[i] cached ones.
// per_tile: queries in a tile; slots: blocks of one KV head that run at once; skip_single: requests that bring
// one token are not this kernel's.  min_tiles: the shortest share worth a block; start_up and unshared: the
// model's constants (cost of one more block, in key tiles; pace of a block whose keys nobody else reads);
// gain: the fraction of the undivided length a division has to get under.
YPOL_API void ypol_kv_splits(const int32_t* q_lens, const int32_t* before, int n_requests, int per_tile, int slots,
                             int skip_single, int min_tiles, double start_up, double unshared, double gain,
                             int32_t* out) {
  out[0] = 1;
  out[1] = 1;
  if (n_requests <= 0 || per_tile <= 0 || slots <= 0) return;
  std::vector<int32_t> tiles;
  std::vector<double> pace;
  int longest = 0;
  for (int i = 0; i < n_requests; ++i) {
    const int q = q_lens[i];
    if (q <= 0 || (skip_single && q == 1)) continue;
    const double p = q <= 3 * per_tile ? unshared : 1.0;
    for (int first = 0; first < q; first += per_tile) {
      const int t = (before[i] + std::min(q, first + per_tile) - 1) / 64 + 1;
      tiles.push_back(t);
      pace.push_back(p);
      longest = std::max(longest, t);
    }
  }
  if (longest < 3 * min_tiles) return;
  const int n = (int)tiles.size();
  double best = gain * step_length(tiles.data(), pace.data(), n, slots, 1, 1, start_up);
  static const int kShares[] = {2, 3, 4, 6, 8};
  for (int shares : kShares) {
    const int limit = std::max(min_tiles, (longest + shares - 1) / shares);
    const double length = step_length(tiles.data(), pace.data(), n, slots, shares, limit, start_up);
    if (length < best) {
      best = length;
      out[0] = std::min(64, (longest + limit - 1) / limit);
      out[1] = limit;
    }
  }
}

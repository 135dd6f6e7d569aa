// Tile-configuration search strategies for the autotuner: grid, random, evolutionary and an
// explore/exploit strategy standing in for the reference's Bayesian search
// (crates/autotuner/src/search.rs: GridSearch :369, RandomSearch, EvolutionarySearch, BayesianSearch).
// The searcher proposes configurations (one choice index per dimension); the caller times the real kernel
// with CUDA events and reports back, so this file has no GPU dependency.
#include <algorithm>
#include <cmath>
#include <limits>
#include <map>
#include <random>
#include <vector>

#include "rb_runtime.h"

struct RbSearch {
  int strategy, max_evals;
  std::vector<std::vector<int>> dims;          // choices per dimension (values)
  std::mt19937_64 rng;
  std::map<std::vector<int>, double> results;  // config (values) -> time
  std::vector<int> best;
  double best_time = std::numeric_limits<double>::infinity();
  long long grid_pos = 0, grid_total = 1;
  int proposed = 0;
  std::vector<std::vector<int>> population;    // evolutionary
  size_t pop_cursor = 0;
  int generation = 0;
};

static std::vector<int> decode_grid(const RbSearch* s, long long idx) {
  std::vector<int> c(s->dims.size());
  for (size_t d = 0; d < s->dims.size(); ++d) {
    c[d] = s->dims[d][idx % (long long)s->dims[d].size()];
    idx /= (long long)s->dims[d].size();
  }
  return c;
}
static std::vector<int> random_config(RbSearch* s) {
  std::vector<int> c(s->dims.size());
  for (size_t d = 0; d < s->dims.size(); ++d) c[d] = s->dims[d][s->rng() % s->dims[d].size()];
  return c;
}
static std::vector<int> mutate(RbSearch* s, std::vector<int> c) {
  const size_t d = s->rng() % s->dims.size();
  c[d] = s->dims[d][s->rng() % s->dims[d].size()];
  return c;
}
static std::vector<int> neighbour(RbSearch* s, const std::vector<int>& c) {
  // move one dimension to an adjacent choice
  std::vector<int> n = c;
  const size_t d = s->rng() % s->dims.size();
  const auto& ch = s->dims[d];
  size_t pos = std::find(ch.begin(), ch.end(), c[d]) - ch.begin();
  if (pos >= ch.size()) pos = 0;
  if (ch.size() > 1) pos = (s->rng() & 1) ? std::min(pos + 1, ch.size() - 1) : (pos == 0 ? 0 : pos - 1);
  n[d] = ch[pos];
  return n;
}

extern "C" {

RbSearch* rb_search_create(int strategy, int num_dims, const int* dim_sizes, const int* choices_flat, uint64_t seed,
                           int max_evals) {
  if (num_dims <= 0 || strategy < 0 || strategy > 3) return nullptr;
  auto* s = new RbSearch;
  s->strategy = strategy;
  s->max_evals = max_evals > 0 ? max_evals : 1 << 30;
  s->rng.seed(seed);
  int off = 0;
  for (int d = 0; d < num_dims; ++d) {
    if (dim_sizes[d] <= 0) { delete s; return nullptr; }
    s->dims.emplace_back(choices_flat + off, choices_flat + off + dim_sizes[d]);
    off += dim_sizes[d];
    s->grid_total *= dim_sizes[d];
  }
  return s;
}
void rb_search_destroy(RbSearch* s) { delete s; }

int rb_search_next(RbSearch* s, int* out) {
  if (s->proposed >= s->max_evals) return 0;
  std::vector<int> c;
  if (s->strategy == 0) {
    if (s->grid_pos >= s->grid_total) return 0;
    c = decode_grid(s, s->grid_pos++);
  } else if (s->strategy == 1) {
    // random without repeats while unseen configurations remain
    if ((long long)s->results.size() >= s->grid_total) return 0;
    int tries = 0;
    do { c = random_config(s); } while (s->results.count(c) && ++tries < 64);
    if (s->results.count(c)) {   // dense spaces: fall back to the first unseen grid point
      for (long long i = 0; i < s->grid_total; ++i) { c = decode_grid(s, i); if (!s->results.count(c)) break; }
    }
  } else if (s->strategy == 2) {
    const size_t pop = 8;
    if (s->population.empty()) for (size_t i = 0; i < pop; ++i) s->population.push_back(random_config(s));
    if (s->pop_cursor >= s->population.size()) {
      // next generation: keep the best half (by reported time), refill with mutations / crossovers of survivors
      std::sort(s->population.begin(), s->population.end(), [&](const std::vector<int>& a, const std::vector<int>& b) {
        auto ia = s->results.find(a), ib = s->results.find(b);
        const double ta = ia == s->results.end() ? 1e300 : ia->second, tb = ib == s->results.end() ? 1e300 : ib->second;
        return ta < tb;
      });
      s->population.resize(pop / 2);
      while (s->population.size() < pop) {
        const auto& p1 = s->population[s->rng() % (pop / 2)];
        const auto& p2 = s->population[s->rng() % (pop / 2)];
        std::vector<int> child(p1.size());
        for (size_t d = 0; d < child.size(); ++d) child[d] = (s->rng() & 1) ? p1[d] : p2[d];
        s->population.push_back(mutate(s, child));
      }
      s->pop_cursor = pop / 2;   // survivors are already measured
      ++s->generation;
    }
    c = s->population[s->pop_cursor++];
  } else {
    // explore (random) for the first quarter of the budget, then exploit neighbours of the incumbent
    const int explore = std::max(4, std::min(s->max_evals, 64) / 4);
    if (s->proposed < explore || s->best.empty()) c = random_config(s);
    else {
      int tries = 0;
      do { c = neighbour(s, s->best); } while (s->results.count(c) && ++tries < 16);
      if (s->results.count(c)) c = random_config(s);
    }
  }
  for (size_t d = 0; d < c.size(); ++d) out[d] = c[d];
  ++s->proposed;
  return 1;
}

void rb_search_report(RbSearch* s, const int* config, double time_us) {
  std::vector<int> c(config, config + s->dims.size());
  auto it = s->results.find(c);
  if (it == s->results.end() || time_us < it->second) s->results[c] = time_us;
  if (time_us < s->best_time) { s->best_time = time_us; s->best = c; }
}

int rb_search_best(const RbSearch* s, int* out, double* t) {
  if (s->best.empty()) return 0;
  for (size_t d = 0; d < s->best.size(); ++d) out[d] = s->best[d];
  if (t) *t = s->best_time;
  return 1;
}
int rb_search_num_evals(const RbSearch* s) { return (int)s->results.size(); }

}  // extern "C"

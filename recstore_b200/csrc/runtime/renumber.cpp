// Id renumbering for "known" cache ranges: the pre-sampled hot ids of rank r receive the new ids
// [start_r, start_r + len_r) with start_r = sum of the previous ranks' hot-set sizes; every other id
// is numbered after all hot sets in increasing old-id order.  After renumbering, rank r's cache is
// simply the id range [start_r, start_r + len_r) (reference: ConstructRenumberingDict,
// src/framework/pytorch/recstore_pytorch.cc:27-62; used by RenumberingGraph,
// src/kg/kg/dgl-ke/python/dglke/dataloader/sampler.py:629-634).
#include <atomic>
#include <vector>

#include "common/rs_common.h"
#include "runtime/base.h"

// dict_out[old_id] = new_id for old_id in [0, n).  hot[r] points at lens[r] distinct old ids; an id may be
// hot on one rank only (a second occurrence is reported as an error).
RS_API int rs_construct_renumbering_dict(long long* dict_out, long long n, int nr_world, const long long* const* hot,
                                         const long long* lens) {
  RS_REQUIRE(dict_out && n >= 0 && nr_world >= 0 && (nr_world == 0 || (hot && lens)), "rs_construct_renumbering_dict: bad argument");
  for (long long i = 0; i < n; ++i) dict_out[i] = -1;
  long long start = 0;
  for (int r = 0; r < nr_world; ++r) {
    for (long long k = 0; k < lens[r]; ++k) {
      const long long id = hot[r][k];
      if (id < 0 || id >= n) return rs::set_error(RS_ERR_INVALID, "hot id %lld of rank %d is outside [0, %lld)", id, r, n);
      if (dict_out[id] != -1) return rs::set_error(RS_ERR_INVALID, "id %lld is hot on more than one rank", id);
      dict_out[id] = start + k;
    }
    start += lens[r];
  }
  // cold ids: prefix count of unassigned entries, in parallel over blocks
  const size_t nb = static_cast<size_t>(rs::ThreadPool::global().size());
  std::vector<long long> cnt(nb + 1, 0);
  const size_t per = (static_cast<size_t>(n) + nb - 1) / nb;
  rs::ThreadPool::global().parallel_for(nb, [&](size_t b0, size_t b1, int) {
    for (size_t b = b0; b < b1; ++b) {
      long long c = 0;
      for (size_t i = b * per; i < std::min(static_cast<size_t>(n), (b + 1) * per); ++i) c += dict_out[i] == -1;
      cnt[b + 1] = c;
    }
  });
  for (size_t b = 0; b < nb; ++b) cnt[b + 1] += cnt[b];
  rs::ThreadPool::global().parallel_for(nb, [&](size_t b0, size_t b1, int) {
    for (size_t b = b0; b < b1; ++b) {
      long long next = start + cnt[b];
      for (size_t i = b * per; i < std::min(static_cast<size_t>(n), (b + 1) * per); ++i)
        if (dict_out[i] == -1) dict_out[i] = next++;
    }
  });
  return RS_OK;
}

// Id generators on the device: the samplers of the benchmarks and of knowledge-graph training draw their ids where they are
// used instead of on the host.
//
//   rs_gen_uniform_ids   uniform ids in [0, range): the negative entities of a KG batch (the reference draws them with
//                        numpy / DGL's sampler on the CPU, src/kg/kg/dgl-ke/python/dglke/dataloader/sampler.py:703-818)
//   rs_gen_zipf_ids      bounded Zipf-like ids for ANY exponent: inverse CDF of the density x^-alpha on [1, range + 1), floored
//                        (same closed form as the host generator, so equal uniforms give equal ids), with an optional affine
//                        permutation (a * k + b) mod range that spreads the popular ids over all shards
//
// Both are counter based: element i of a call draws from hash(seed, counter + i), so a stream is reproducible, independent of
// the launch shape, and two calls with disjoint counter ranges never repeat a draw.
#include "common/rs_common.h"

namespace {

__host__ __device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}
__device__ __forceinline__ unsigned long long draw(unsigned long long seed, unsigned long long ctr) {
  return splitmix64(splitmix64(seed) ^ (ctr * 0xD1342543DE82EF95ull + 0x2545F4914F6CDD1Dull));
}

__global__ void gen_uniform_kernel(long long* __restrict__ out, long long n, unsigned long long range, unsigned long long seed,
                                   unsigned long long counter) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x)
    out[i] = static_cast<long long>(__umul64hi(draw(seed, counter + i), range));   // floor(u * range), u in [0, 1)
}

__global__ void gen_zipf_kernel(long long* __restrict__ out, long long n, unsigned long long range, double alpha, unsigned long long seed,
                                unsigned long long counter, unsigned long long perm_a, unsigned long long perm_b) {
  const double n1 = static_cast<double>(range) + 1.0;
  const bool is_one = fabs(alpha - 1.0) < 1e-9;
  const double e = 1.0 - alpha;
  const double c = is_one ? log(n1) : pow(n1, e) - 1.0;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const double u = static_cast<double>(draw(seed, counter + i) >> 11) * (1.0 / 9007199254740992.0);   // 53 bits -> [0, 1)
    const double x = is_one ? exp(u * c) : pow(u * c + 1.0, 1.0 / e);
    long long k = static_cast<long long>(floor(x)) - 1;
    if (k < 0) k = 0;
    if (k >= static_cast<long long>(range)) k = static_cast<long long>(range) - 1;
    if (perm_a) {
      // (a * k + b) mod range without overflow: 128-bit product through the high / low halves
      const unsigned long long lo = perm_a * static_cast<unsigned long long>(k);
      const unsigned long long hi = __umul64hi(perm_a, static_cast<unsigned long long>(k));
      unsigned long long r = hi % range;
      // r * 2^64 mod range, 8 bits at a time
      for (int s = 0; s < 8; ++s) r = ((r << 8) % range);
      r = (r + lo % range) % range;
      k = static_cast<long long>((r + perm_b % range) % range);
    }
    out[i] = k;
  }
}

int grid_of(long long n) {
  long long g = (n + 255) / 256;
  if (g > 148 * 8) g = 148 * 8;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}
}  // namespace

RS_API int rs_gen_uniform_ids(long long* out, long long n, long long range, unsigned long long seed, unsigned long long counter,
                              cudaStream_t stream) {
  RS_REQUIRE(out && n >= 0 && range > 0, "rs_gen_uniform_ids: bad argument");
  if (n == 0) return RS_OK;
  gen_uniform_kernel<<<grid_of(n), 256, 0, stream>>>(out, n, static_cast<unsigned long long>(range), seed, counter);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

// perm_a = 0: ids in popularity order (0 is the hottest); otherwise id = (perm_a * k + perm_b) mod range, perm_a coprime to range.
// range < 2^56 (the permutation reduces 64-bit words 8 bits at a time).
RS_API int rs_gen_zipf_ids(long long* out, long long n, long long range, double alpha, unsigned long long seed,
                           unsigned long long counter, unsigned long long perm_a, unsigned long long perm_b, cudaStream_t stream) {
  RS_REQUIRE(out && n >= 0 && range > 0 && range < (1ll << 56) && alpha >= 0.0, "rs_gen_zipf_ids: bad argument");
  if (n == 0) return RS_OK;
  gen_zipf_kernel<<<grid_of(n), 256, 0, stream>>>(out, n, static_cast<unsigned long long>(range), alpha, seed, counter, perm_a, perm_b);
  RS_LAUNCH_CHECK();
  return RS_OK;
}

// The uniform that element `ctr` of a stream draws (host mirror for tests and for host-side replays of a device stream).
RS_API unsigned long long rs_gen_draw(unsigned long long seed, unsigned long long ctr) {
  return splitmix64(splitmix64(seed) ^ (ctr * 0xD1342543DE82EF95ull + 0x2545F4914F6CDD1Dull));
}

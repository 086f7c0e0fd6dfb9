// Host-side KV engines behind one interface, created by name through a factory.
//
// Interface and semantics follow BaseKV of the reference (src/storage/kv_engine/base_kv.h:19-56:
// Get, Put, BatchGet, BatchPut, BulkLoad, clear, DebugInfo, created from a json_config with
// path / capacity / value_size) and its string-keyed factory (engine_map.h:129,
// kv_engine_register.cc:1-11).  Values are fixed-size byte strings (value_size from the config).
// Engines:
//   "KVEngineMap"            sharded unordered_map + reader/writer locks (engine_map.h:10-129)
//   "KVEngineExtendibleHash" extendible hashing with bucket splits and directory doubling
//                            (engine_extendiblehash.h:12-130, dram/src/extendible_hash.cpp)
//   "KVEnginePoolMap"        sharded index over out-of-place sealed records in a crash-recoverable slab pool,
//                            readers protected by epochs (kv_engine_pool.cpp, persist_pool.h)
//   "KVEngineChunkHash"      14-slot tagged chunks with SSE2 tag matching and overflow counters,
//                            16 shards, optional file-backed persistence with crash reload and
//                            hot-key migration (role of PetHash / PetKV, nvm/pet_kv/pet_hash.h:
//                            45-117, 154-249, 422-510)
// The first three engines store values in a SlabValueStore (bump allocator + free list over an anonymous or
// file-backed mapping; role of PersistSimpleMalloc, src/memory/persist_malloc.h:26-124).
#pragma once
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

namespace rs {

struct KVConfig {
  std::string path;          // empty = volatile; else directory for the engine's files
  uint64_t capacity = 1 << 20;
  uint32_t value_size = 128;
  int num_threads = 8;
  int num_shards = 64;
  bool prefetch = false;
  std::string raw_json;
};

class BaseKV {
 public:
  virtual ~BaseKV() = default;
  // Copies the value into out (value_size bytes).  Returns false when the key is absent.
  virtual bool Get(uint64_t key, void* out) = 0;
  virtual bool Put(uint64_t key, const void* value) = 0;   // false: engine full
  virtual bool Erase(uint64_t key) = 0;
  // found[i] = 1/0; absent keys leave out[i] zero-filled.
  virtual void BatchGet(const uint64_t* keys, size_t n, void* out, uint8_t* found);
  virtual size_t BatchPut(const uint64_t* keys, size_t n, const void* values);  // returns #stored
  // key i in [0, n) -> value = float(key) repeated (the reference's LoadFakeData / BulkLoad pattern).
  virtual void BulkLoad(uint64_t n);
  virtual void Clear() = 0;
  virtual uint64_t Size() const = 0;
  virtual std::string DebugInfo() const = 0;
  virtual bool Persistent() const { return false; }
  virtual void Flush() {}
  // Enumerates up to cap keys (checkpointing); returns the number written.
  virtual size_t Keys(uint64_t* out, size_t cap) const = 0;
  uint32_t value_size() const { return cfg_.value_size; }
  const KVConfig& config() const { return cfg_; }

 protected:
  explicit BaseKV(const KVConfig& c) : cfg_(c) {}
  KVConfig cfg_;
};

// Factory: returns nullptr and sets rs::set_error for unknown names.
std::unique_ptr<BaseKV> CreateKV(const std::string& engine, const KVConfig& cfg);
std::vector<std::string> ListKVEngines();
KVConfig ParseKVConfig(const std::string& json);

}  // namespace rs

// Drop-in for llm-engine's include/engine/kv_cache.h: put this repository's
// include/ directory ahead of llm-engine's on the include path and
// `#include "engine/kv_cache.h"` resolves here, giving engine::KVCacheManager,
// engine::BlockTable, engine::BlockId, engine::kNoBlock and engine::KVCacheStats
// backed by the implementation in libpkv (include/pkv_kv_cache.hpp).
#pragma once
#include "../pkv_kv_cache.hpp"

namespace engine {
using pkv::BlockId;
using pkv::BlockTable;
using pkv::kNoBlock;
using pkv::KVCacheManager;
using pkv::KVCacheStats;
}  // namespace engine

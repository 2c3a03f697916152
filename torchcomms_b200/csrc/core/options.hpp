// Communicator and per-operation options, environment parsing helpers.
//
// Parity: comms/torchcomms/TorchCommOptions.hpp:20-89 (option structs, typed
// hint lookup, env defaults TORCHCOMM_ABORT_ON_ERROR / TORCHCOMM_TIMEOUT_SECONDS)
// and comms/torchcomms/utils/Utils.cpp:58-216 (env_to_value, rank/size probing).
#pragma once

#include <c10/util/intrusive_ptr.h>
#include <torch/csrc/distributed/c10d/Store.hpp>

#include <array>
#include <sstream>
#include <vector>
#include <type_traits>

#include "types.hpp"

namespace b200c {

B200C_API bool parse_bool(std::string_view text);

// Configuration tiers (comms/utils/cvars/README.md:10-19 has the same order for
// the reference's knobs): the environment wins, then the configuration file
// (`B200COMMS_CONF_FILE`, default /etc/b200comms.conf; lines `KEY=VALUE`, `#`
// comments), then the built-in default. Returns nullptr when neither tier has
// the key; `*source` becomes "env" or "file".
B200C_API const char* config_raw(const char* key, const char** source = nullptr);
// Forgets the parsed configuration file so the next lookup reads it again.
B200C_API void reload_config_file();
// Every key looked up so far with the value in force and where it came from
// ("env", "file" or "default"), for `knobs()` in Python.
B200C_API void note_knob(const char* key, const std::string& value, const char* source);
B200C_API std::vector<std::array<std::string, 3>> knob_report();

template <typename T>
std::string knob_text(const T& v) {
  if constexpr (std::is_same_v<T, std::string>) {
    return v;
  } else {
    std::ostringstream o;
    o << v;
    return o.str();
  }
}

// Reads a configuration key (environment, then configuration file) and converts
// it; returns `fallback` when the key is unset or empty. Throws
// std::runtime_error on malformed values.
template <typename T>
T env_to_value(const char* key, const T& fallback) {
  const char* source = "default";
  const char* raw = config_raw(key, &source);
  if (raw == nullptr || *raw == '\0') {
    note_knob(key, knob_text(fallback), "default");
    return fallback;
  }
  note_knob(key, raw, source);
  if constexpr (std::is_same_v<T, bool>) {
    return parse_bool(raw);
  } else if constexpr (std::is_same_v<T, std::string>) {
    return std::string(raw);
  } else {
    std::istringstream in(raw);
    T out{};
    in >> out;
    if (in.fail() || !in.eof()) {
      throw std::runtime_error(
          std::string("cannot parse environment variable ") + key + "='" + raw + "'");
    }
    return out;
  }
}

// Typed lookup in a hints dictionary with a fallback.
template <typename T>
T hint_or(const Hints& hints, const std::string& key, const T& fallback) {
  auto it = hints.find(key);
  if (it == hints.end()) {
    return fallback;
  }
  if constexpr (std::is_same_v<T, bool>) {
    return parse_bool(it->second);
  } else if constexpr (std::is_same_v<T, std::string>) {
    return it->second;
  } else {
    std::istringstream in(it->second);
    T out{};
    in >> out;
    if (in.fail()) {
      throw std::runtime_error("cannot parse hint " + key + "='" + it->second + "'");
    }
    return out;
  }
}

// Options common to every single operation.
struct OpOptions {
  Hints hints;
  Millis timeout{kDefaultTimeout};
  bool timeout_set = false; // false: inherit the communicator's timeout
};

struct B200C_API CommOptions {
  CommOptions();
  bool abort_process_on_timeout_or_error;
  Millis timeout;
  bool is_high_priority_stream = false;
  c10::intrusive_ptr<c10d::Store> store;
  bool enable_reconfigure = false;
  Hints hints;
  std::string name;   // the communicator's name; filled in by new_comm() / split() for backends that read it here
};

struct ReconfigureOptions {
  int64_t uuid = 0;
  std::vector<InitHandle> handles;
  bool handles_ordered = true; // a list fixes rank order; a set sorts handles
  std::optional<Millis> timeout;
  Hints hints;
};

// Rank and world size discovered from the launcher's environment. The probe
// order is TORCHCOMM_RANK/SIZE, Open MPI, PMI, PALS, torchrun; the variable
// TORCHCOMM_BOOTSTRAP_RANKSIZE_QUERY_METHOD pins one of
// {auto, torchcomm, ompi, pmi, pals, torchrun}.
std::pair<int, int> query_ranksize();

// A TCPStore at MASTER_ADDR:MASTER_PORT (rank 0 hosts it) wrapped in a
// PrefixStore scoped by `prefix`.
c10::intrusive_ptr<c10d::Store> create_prefix_store(
    const std::string& prefix,
    int rank,
    int world_size,
    Millis timeout);

// A second TCPStore of its own (rank 0 listens on a port the system picks and
// publishes it through `bootstrap` under "<prefix>/dup_store_port"), wrapped
// in a PrefixStore. For users that must not share a server with the bootstrap
// store (comms/torchcomms/utils/StoreManager.cpp:37-80).
c10::intrusive_ptr<c10d::Store> dup_prefix_store(
    const std::string& prefix,
    const c10::intrusive_ptr<c10d::Store>& bootstrap,
    Millis timeout);

// Wraps an existing store so keys of one communicator cannot collide with
// another's.
c10::intrusive_ptr<c10d::Store> scoped_store(
    const c10::intrusive_ptr<c10d::Store>& base,
    const std::string& prefix);

// Small helpers on top of a c10d store.
void store_set_string(c10d::Store& s, const std::string& key, const std::string& v);
std::string store_get_string(c10d::Store& s, const std::string& key);
// Counts arrivals under `key`; returns once `world` ranks have arrived.
void store_barrier(c10d::Store& s, const std::string& key, int rank, int world, Millis timeout);

} // namespace b200c

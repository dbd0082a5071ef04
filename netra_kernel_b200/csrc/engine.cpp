// Netra engine runtime for sm_100a: loads an engine directory written by the compiler, binds
// caller-owned pointers, optionally captures a CUDA graph, and launches on the caller's stream.
//
// Behavioural contract followed: runtime/gfx950/engine/netra_engine.hip:249-566 (create / query /
// bind / finalize / prepare / launch / launch_operation / launch_operation_bound / destroy) with
// its status codes, ordering rules and hot-path rules (no allocation, synchronisation, file, env
// or string work in the launch functions).  Kernels come from cubins through the CUDA driver API,
// reached through cudaGetDriverEntryPoint so that the library has no link-time libcuda dependency.
#include <cuda.h>
#include <cuda_runtime_api.h>

#include <array>
#include <atomic>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <functional>
#include <limits>
#include <map>
#include <memory>
#include <mutex>
#include <new>
#include <sstream>
#include <stdexcept>
#include <string>
#include <tuple>
#include <vector>

#include "../../include/netra_engine.h"

namespace {

// ----------------------------------------------------------------------------- JSON
struct Json {
  enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
  bool boolean = false;
  uint64_t number = 0;      // manifests only carry non-negative integers
  bool integral = true;
  std::string string;
  std::vector<Json> array;
  std::vector<std::pair<std::string, Json>> object;

  const Json* find(const char* key) const {
    if (kind != Object) return nullptr;
    for (const auto& kv : object)
      if (kv.first == key) return &kv.second;
    return nullptr;
  }
  const Json& at(const char* key) const {
    const Json* v = find(key);
    if (!v) throw std::runtime_error(std::string("missing manifest field: ") + key);
    return *v;
  }
};

class JsonReader {
 public:
  explicit JsonReader(const std::string& text) : t_(text) {}
  Json parse() {
    Json v = value(0);
    space();
    if (p_ != t_.size()) fail("trailing characters after JSON value");
    return v;
  }

 private:
  const std::string& t_;
  size_t p_ = 0;
  [[noreturn]] void fail(const char* what) const {
    throw std::runtime_error(std::string("engine.json: ") + what + " at byte " + std::to_string(p_));
  }
  void space() { while (p_ < t_.size() && (t_[p_] == ' ' || t_[p_] == '\n' || t_[p_] == '\t' || t_[p_] == '\r')) ++p_; }
  bool take(char c) { space(); if (p_ < t_.size() && t_[p_] == c) { ++p_; return true; } return false; }
  void expect(char c) { if (!take(c)) fail("unexpected character"); }
  Json value(int depth) {
    if (depth > 64) fail("nesting too deep");
    space();
    if (p_ >= t_.size()) fail("unexpected end");
    const char c = t_[p_];
    Json v;
    if (c == '{') {
      ++p_; v.kind = Json::Object;
      if (take('}')) return v;
      do {
        space();
        Json key = string_value();
        expect(':');
        v.object.emplace_back(key.string, value(depth + 1));
      } while (take(','));
      expect('}');
    } else if (c == '[') {
      ++p_; v.kind = Json::Array;
      if (take(']')) return v;
      do { v.array.push_back(value(depth + 1)); } while (take(','));
      expect(']');
    } else if (c == '"') {
      v = string_value();
    } else if (c == 't' && t_.compare(p_, 4, "true") == 0) {
      p_ += 4; v.kind = Json::Bool; v.boolean = true;
    } else if (c == 'f' && t_.compare(p_, 5, "false") == 0) {
      p_ += 5; v.kind = Json::Bool;
    } else if (c == 'n' && t_.compare(p_, 4, "null") == 0) {
      p_ += 4;
    } else {
      v.kind = Json::Number;
      const size_t begin = p_;
      if (t_[p_] == '-') { v.integral = false; ++p_; }
      uint64_t n = 0; bool any = false;
      while (p_ < t_.size() && t_[p_] >= '0' && t_[p_] <= '9') {
        const uint64_t d = (uint64_t)(t_[p_] - '0');
        if (n > (std::numeric_limits<uint64_t>::max() - d) / 10) fail("integer overflows uint64");
        n = n * 10 + d; any = true; ++p_;
      }
      if (!any) fail("invalid value");
      if (p_ < t_.size() && (t_[p_] == '.' || t_[p_] == 'e' || t_[p_] == 'E')) {
        v.integral = false;
        while (p_ < t_.size() && (std::strchr("+-.eE", t_[p_]) || (t_[p_] >= '0' && t_[p_] <= '9'))) ++p_;
      }
      v.number = n;
      (void)begin;
    }
    return v;
  }
  Json string_value() {
    if (p_ >= t_.size() || t_[p_] != '"') fail("expected string");
    ++p_;
    Json v; v.kind = Json::String;
    while (p_ < t_.size() && t_[p_] != '"') {
      char c = t_[p_++];
      if (c == '\\') {
        if (p_ >= t_.size()) fail("bad escape");
        const char e = t_[p_++];
        switch (e) {
          case 'n': c = '\n'; break; case 't': c = '\t'; break; case 'r': c = '\r'; break;
          case 'b': c = '\b'; break; case 'f': c = '\f'; break;
          case '"': case '\\': case '/': c = e; break;
          case 'u': {
            if (p_ + 4 > t_.size()) fail("bad unicode escape");
            unsigned code = 0;
            for (int i = 0; i < 4; ++i) {
              const char h = t_[p_++];
              code = code * 16 + (unsigned)(h >= '0' && h <= '9' ? h - '0' : (h | 32) >= 'a' && (h | 32) <= 'f' ? (h | 32) - 'a' + 10 : 99);
            }
            if (code > 0x7f) fail("non-ASCII escape is not supported in engine manifests");
            c = (char)code; break;
          }
          default: fail("bad escape");
        }
      }
      v.string.push_back(c);
    }
    if (p_ >= t_.size()) fail("unterminated string");
    ++p_;
    return v;
  }
};

uint32_t as_u32(const Json& v, const char* name) {
  if (v.kind != Json::Number || !v.integral || v.number > UINT32_MAX) throw std::runtime_error(std::string(name) + " must be uint32");
  return (uint32_t)v.number;
}
uint64_t as_u64(const Json& v, const char* name) {
  if (v.kind != Json::Number || !v.integral) throw std::runtime_error(std::string(name) + " must be uint64");
  return v.number;
}
const std::string& as_text(const Json& v, const char* name) {
  if (v.kind != Json::String) throw std::runtime_error(std::string(name) + " must be a string");
  return v.string;
}

// A file of the engine directory could not be read (reported as NETRA_STATUS_IO, not as a malformed manifest).
struct IoFailure : std::runtime_error {
  using std::runtime_error::runtime_error;
};

std::string read_file(const std::string& path) {
  std::ifstream in(path, std::ios::binary);
  if (!in) throw IoFailure("cannot open " + path);
  std::ostringstream ss; ss << in.rdbuf();
  return ss.str();
}

// "cubin/<name>" only: no absolute paths, backslashes, empty or dot components.
std::string checked_cubin_path(const std::string& rel) {
  if (rel.rfind("cubin/", 0) != 0 || rel.size() <= 6 || rel.find('\\') != std::string::npos || rel.find("//") != std::string::npos)
    throw std::runtime_error("cubin must be a normalized engine-relative path");
  size_t begin = 0;
  while (begin <= rel.size()) {
    const size_t end = rel.find('/', begin);
    const std::string part = rel.substr(begin, end == std::string::npos ? std::string::npos : end - begin);
    if (part.empty() || part == "." || part == "..") throw std::runtime_error("cubin path traversal is forbidden");
    if (end == std::string::npos) break;
    begin = end + 1;
  }
  return rel;
}

std::pair<uint32_t, uint32_t> major_minor(const std::string& text) {
  const size_t dot = text.find('.');
  if (dot == std::string::npos || dot == 0 || dot + 1 == text.size() || text.find('.', dot + 1) != std::string::npos)
    throw std::runtime_error("required_cuda.minimum must be MAJOR.MINOR");
  for (char c : text)
    if (c != '.' && (c < '0' || c > '9')) throw std::runtime_error("required_cuda.minimum must be MAJOR.MINOR");
  const unsigned long a = std::stoul(text.substr(0, dot)), b = std::stoul(text.substr(dot + 1));
  if (a > 1000 || b > 1000) throw std::runtime_error("required_cuda.minimum is out of range");
  return {(uint32_t)a, (uint32_t)b};
}

// ----------------------------------------------------------------------------- manifest model
constexpr uint32_t kMaxArguments = 32;

struct TensorMapSpec {
  uint64_t rows = 0, row_bytes = 0;
  uint32_t box_rows = 0, box_bytes = 0;
  bool four_bit = false;   // element "e2m1": rows of 128 four-bit codes (64 bytes in memory) widened to 128 bytes of shared memory
};

struct ArgSpec {
  enum Kind { Pointer, U32, TensorMap } kind = Pointer;
  bool bindable = false;          // source == binding
  bool null_pointer = false;      // source == null: an optional operand the model does not have
  uint64_t workspace_offset = 0;  // source == workspace
  uint32_t value = 0;             // u32_constant
  TensorMapSpec map;
};

struct OpSpec {
  bool fallback = true;
  uint32_t grid[3] = {1, 1, 1}, block[3] = {1, 1, 1}, lds_bytes = 0, dynamic_lds_bytes = 0;
  uint32_t registers_per_thread = 0;   // nonzero: the code object must report exactly this allocation
  std::string cubin, symbol;
  std::vector<ArgSpec> args;
};

struct ProfileSpec {
  netra_profile_info_t info{};
};

struct Manifest {
  uint64_t workspace_bytes = 0;
  std::pair<uint32_t, uint32_t> required_cuda{0, 0};
  std::vector<ProfileSpec> profiles;
  std::vector<OpSpec> operations;
};

Manifest parse_manifest(const std::string& directory) {
  const Json root = JsonReader(read_file(directory + "/engine.json")).parse();
  if (as_text(root.at("format_version"), "format_version") != "netra-engine-1" ||
      as_text(root.at("target"), "target") != "sm_100a" || as_u32(root.at("wave_size"), "wave_size") != 32)
    throw std::runtime_error("engine target/format/wave contract mismatch");
  Manifest m;
  m.required_cuda = major_minor(as_text(root.at("required_cuda").at("minimum"), "required_cuda.minimum"));
  m.workspace_bytes = as_u64(root.at("workspace_bytes"), "workspace_bytes");
  const Json& profiles = root.at("profiles");
  const Json& operations = root.at("operations");
  if (profiles.kind != Json::Array || operations.kind != Json::Array) throw std::runtime_error("profiles and operations must be arrays");
  if (profiles.array.empty()) throw std::runtime_error("engine has no profile");
  for (const Json& op : operations.array) {
    OpSpec spec;
    spec.fallback = as_text(op.at("execution"), "execution") != "kernel";
    const Json* launch = op.find("launch");
    if (launch && launch->kind == Json::Object) {
      const Json& grid = launch->at("grid");
      const Json& block = launch->at("block");
      if (grid.kind != Json::Array || block.kind != Json::Array || grid.array.size() != 3 || block.array.size() != 3)
        throw std::runtime_error("launch grid and block must have three dimensions");
      for (int i = 0; i < 3; ++i) {
        spec.grid[i] = as_u32(grid.array[i], "grid");
        spec.block[i] = as_u32(block.array[i], "block");
        if (!spec.grid[i] || !spec.block[i]) throw std::runtime_error("launch dimensions must be nonzero");
      }
      spec.lds_bytes = as_u32(launch->at("lds_bytes"), "lds_bytes");
      const Json* dyn = launch->find("dynamic_lds_bytes");
      spec.dynamic_lds_bytes = dyn ? as_u32(*dyn, "dynamic_lds_bytes") : 0;
      const Json* regs = launch->find("registers_per_thread");
      spec.registers_per_thread = regs ? as_u32(*regs, "registers_per_thread") : 0;
    } else if (!spec.fallback) {
      throw std::runtime_error("selected kernel requires a launch record");
    }
    if (!spec.fallback) {
      spec.cubin = checked_cubin_path(as_text(op.at("cubin"), "cubin"));
      spec.symbol = as_text(op.at("kernel_symbol"), "kernel_symbol");
      const Json& args = op.at("arguments");
      if (args.kind != Json::Array || args.array.empty()) throw std::runtime_error("selected kernel requires typed arguments");
      if (args.array.size() > kMaxArguments) throw std::runtime_error("more than 32 kernel arguments");
      for (const Json& a : args.array) {
        ArgSpec arg;
        const std::string& kind = as_text(a.at("kind"), "argument.kind");
        if (kind == "pointer" || kind == "tensor_map") {
          arg.kind = kind == "pointer" ? ArgSpec::Pointer : ArgSpec::TensorMap;
          const Json* source = a.find("source");
          const std::string src = source ? as_text(*source, "argument.source") : "binding";
          if (src == "binding") {
            arg.bindable = true;
          } else if (src == "workspace") {
            arg.workspace_offset = as_u64(a.at("workspace_offset"), "workspace_offset");
            if (arg.workspace_offset >= m.workspace_bytes) throw std::runtime_error("kernel workspace argument is out of range");
          } else if (src == "null" && arg.kind == ArgSpec::Pointer) {
            arg.null_pointer = true;
          } else {
            throw std::runtime_error("unsupported pointer argument source: " + src);
          }
          if (arg.kind == ArgSpec::TensorMap) {
            const Json& t = a.at("tensor_map");
            arg.map.rows = as_u64(t.at("rows"), "tensor_map.rows");
            arg.map.row_bytes = as_u64(t.at("row_bytes"), "tensor_map.row_bytes");
            arg.map.box_rows = as_u32(t.at("box_rows"), "tensor_map.box_rows");
            arg.map.box_bytes = as_u32(t.at("box_bytes"), "tensor_map.box_bytes");
            if (t.find("element") != nullptr) {
              const std::string element = as_text(t.at("element"), "tensor_map.element");
              if (element != "u8" && element != "e2m1") throw std::runtime_error("unsupported tensor_map element");
              arg.map.four_bit = element == "e2m1";
            }
            if (as_text(t.at("swizzle"), "tensor_map.swizzle") != "128B" || arg.map.box_bytes != 128 || !arg.map.rows ||
                !arg.map.row_bytes || arg.map.row_bytes % 16 || !arg.map.box_rows || arg.map.box_rows > 256 ||
                (arg.map.four_bit && arg.map.row_bytes != 64))
              throw std::runtime_error("unsupported tensor_map description");
            if (!arg.bindable && arg.workspace_offset % 16) throw std::runtime_error("tensor_map workspace offset must be 16-byte aligned");
          }
        } else if (kind == "u32_constant") {
          arg.kind = ArgSpec::U32;
          arg.value = as_u32(a.at("value"), "argument.value");
        } else {
          throw std::runtime_error("unsupported kernel argument kind: " + kind);
        }
        spec.args.push_back(arg);
      }
    }
    m.operations.push_back(std::move(spec));
  }
  uint32_t id = 0;
  for (const Json& p : profiles.array) {
    ProfileSpec spec;
    const Json& guards = p.at("guards");
    spec.info.struct_size = sizeof(spec.info);
    spec.info.profile_id = id++;
    spec.info.min_m = as_u32(guards.at("m").at("min"), "m.min");
    spec.info.max_m = as_u32(guards.at("m").at("max"), "m.max");
    spec.info.min_batch = as_u32(guards.at("batch").at("min"), "batch.min");
    spec.info.max_batch = as_u32(guards.at("batch").at("max"), "batch.max");
    spec.info.min_sequence = as_u64(guards.at("sequence").at("min"), "sequence.min");
    spec.info.max_sequence = as_u64(guards.at("sequence").at("max"), "sequence.max");
    spec.info.tensor_parallel = as_u32(p.at("tensor_parallel"), "tensor_parallel");
    spec.info.workspace_bytes = m.workspace_bytes;
    for (const OpSpec& op : m.operations)
      if (op.fallback) spec.info.requires_fallback = 1;
    m.profiles.push_back(spec);
  }
  return m;
}

// ----------------------------------------------------------------------------- driver entry points
struct Driver {
  CUresult (*ModuleLoadData)(CUmodule*, const void*) = nullptr;
  CUresult (*ModuleUnload)(CUmodule) = nullptr;
  CUresult (*ModuleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
  CUresult (*FuncSetAttribute)(CUfunction, CUfunction_attribute, int) = nullptr;
  CUresult (*FuncGetAttribute)(int*, CUfunction_attribute, CUfunction) = nullptr;
  CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream,
                           void**, void**) = nullptr;
  CUresult (*TensorMapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill) = nullptr;
  bool ok = false;
};

const Driver& driver() {
  static Driver d = [] {
    Driver r;
    auto get = [](const char* name, void** out) {
      cudaDriverEntryPointQueryResult q;
      return cudaGetDriverEntryPoint(name, out, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess && *out;
    };
    r.ok = get("cuModuleLoadData", (void**)&r.ModuleLoadData) && get("cuModuleUnload", (void**)&r.ModuleUnload) &&
           get("cuModuleGetFunction", (void**)&r.ModuleGetFunction) && get("cuFuncSetAttribute", (void**)&r.FuncSetAttribute) &&
           get("cuFuncGetAttribute", (void**)&r.FuncGetAttribute) &&
           get("cuLaunchKernel", (void**)&r.LaunchKernel) && get("cuTensorMapEncodeTiled", (void**)&r.TensorMapEncodeTiled);
    return r;
  }();
  return d;
}

bool encode_map(CUtensorMap* map, void* base, const TensorMapSpec& s) {
  if (s.four_bit) {   // 128 codes per row, 64 bytes apart in memory; the base must be 32-byte aligned
    cuuint64_t dims[2] = {128, s.rows};
    cuuint64_t strides[1] = {64};
    cuuint32_t box[2] = {128, s.box_rows};
    cuuint32_t elem[2] = {1, 1};
    return ((uintptr_t)base & 31) == 0 &&
           driver().TensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 2, base, dims, strides, box, elem,
                                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  }
  cuuint64_t dims[2] = {s.row_bytes, s.rows};
  cuuint64_t strides[1] = {s.row_bytes};
  cuuint32_t box[2] = {s.box_bytes, s.box_rows};
  cuuint32_t elem[2] = {1, 1};
  return driver().TensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, dims, strides, box, elem,
                                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// ----------------------------------------------------------------------------- engine records
struct ArgSlot {
  ArgSpec spec;
  void* pointer = nullptr;            // bound or workspace-resolved pointer
  uint32_t scalar = 0;
  alignas(64) CUtensorMap map;
  bool map_ready = false;
};

struct OpRecord {
  OpSpec spec;
  CUfunction function = nullptr;
  uint32_t argc = 0;
  std::unique_ptr<ArgSlot[]> slots;   // allocated at create; never resized afterwards
  void* addresses[kMaxArguments] = {};
};

struct ProfileRecord {
  netra_profile_info_t info{};
  std::vector<OpRecord> operations;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t graph_exec = nullptr;
  bool graph_prepared = false;
};

}  // namespace

struct netra_engine {
  std::string directory;
  int device_id = 0;
  bool graph_enabled = false;
  void* workspace = nullptr;
  uint64_t workspace_bytes = 0;
  std::vector<ProfileRecord> profiles;
  std::map<std::string, CUmodule> modules;
  std::atomic<bool> bindings_finalized{false};
  std::atomic<uint32_t> in_flight{0};
  std::array<char, 512> last_error{};
};

namespace {

// ---- error reporting ------------------------------------------------------------------------------
// Every refusal is a (status, text) pair; the text goes to the engine's 512-byte buffer when there is an engine.
netra_status_t refuse(netra_engine* e, netra_status_t status, const char* text) {
  if (e) std::snprintf(e->last_error.data(), e->last_error.size(), "%s", text);
  return status;
}
netra_status_t runtime_error(netra_engine* e, const char* call, cudaError_t err) {
  if (e) std::snprintf(e->last_error.data(), e->last_error.size(), "%s returned %s", call, cudaGetErrorString(err));
  return NETRA_STATUS_CUDA;
}
netra_status_t driver_error(netra_engine* e, const char* call, CUresult err) {
  if (e) std::snprintf(e->last_error.data(), e->last_error.size(), "%s returned CUresult %d", call, (int)err);
  return NETRA_STATUS_CUDA;
}
void clear_error(netra_engine* e) { e->last_error[0] = '\0'; }

// A failure while an engine is being built: carries the status the caller will see.  The text outlives the
// half-built engine in a thread-local buffer (netra_engine_create_error).
struct CreateFailure {
  netra_status_t status;
  std::string text;
};
thread_local std::array<char, 512> g_create_error{};

[[noreturn]] void create_fail(netra_status_t status, const std::string& text) { throw CreateFailure{status, text}; }

// ---- launching -------------------------------------------------------------------------------------
// Counts a caller as being inside a launch entry point for as long as the object lives (destroy answers BUSY meanwhile).
class InFlight {
 public:
  explicit InFlight(netra_engine* e) : e_(e) { e_->in_flight.fetch_add(1, std::memory_order_acq_rel); }
  ~InFlight() { e_->in_flight.fetch_sub(1, std::memory_order_acq_rel); }
  InFlight(const InFlight&) = delete;
  InFlight& operator=(const InFlight&) = delete;

 private:
  netra_engine* e_;
};

bool shape_within(const netra_profile_info_t& g, const netra_launch_shape_t& s) {
  const bool m_ok = g.min_m <= s.m && s.m <= g.max_m;
  const bool batch_ok = g.min_batch <= s.batch && s.batch <= g.max_batch;
  const bool seq_ok = g.min_sequence <= s.sequence && s.sequence <= g.max_sequence;
  return m_ok && batch_ok && seq_ok && s.tensor_parallel == g.tensor_parallel;
}

// What all three launch entry points establish first: the arguments name a profile (and an operation) of this engine, the
// calling thread's current device is the engine's, and the shape passes the profile's guards.
struct LaunchContext {
  ProfileRecord* profile = nullptr;
  OpRecord* op = nullptr;     // only for the per-operation entry points
};

netra_status_t open_launch(netra_engine* e, uint32_t profile_id, const uint32_t* operation_index, const netra_launch_shape_t* shape,
                           LaunchContext* ctx) {
  if (!e || !shape || profile_id >= e->profiles.size()) return NETRA_STATUS_INVALID_ARGUMENT;
  ProfileRecord& profile = e->profiles[profile_id];
  if (operation_index && *operation_index >= profile.operations.size()) return NETRA_STATUS_INVALID_ARGUMENT;
  int current = -1;
  const cudaError_t err = cudaGetDevice(&current);
  if (err != cudaSuccess) return runtime_error(e, "cudaGetDevice", err);
  if (current != e->device_id)
    return refuse(e, NETRA_STATUS_UNSUPPORTED_TARGET, "the calling thread's current device is not the device this engine was created on");
  if (!shape_within(profile.info, *shape))
    return refuse(e, NETRA_STATUS_UNSUPPORTED_PROFILE, "launch shape is outside this profile's m / batch / sequence / tensor-parallel guards");
  ctx->profile = &profile;
  ctx->op = operation_index ? &profile.operations[*operation_index] : nullptr;
  return NETRA_STATUS_OK;
}

netra_status_t launch_record(netra_engine* e, OpRecord& op, void** addresses, cudaStream_t stream) {
  const OpSpec& k = op.spec;
  const CUresult r = driver().LaunchKernel(op.function, k.grid[0], k.grid[1], k.grid[2], k.block[0], k.block[1], k.block[2],
                                           k.dynamic_lds_bytes, (CUstream)stream, addresses, nullptr);
  return r == CUDA_SUCCESS ? NETRA_STATUS_OK : driver_error(e, "cuLaunchKernel", r);
}

bool has_unbound_slot(const OpRecord& op) {
  for (uint32_t i = 0; i < op.argc; ++i)
    if (op.slots[i].spec.bindable && op.slots[i].pointer == nullptr) return true;
  return false;
}

netra_status_t launch_one(netra_engine* e, OpRecord& op, cudaStream_t stream) {
  if (op.spec.fallback) return refuse(e, NETRA_STATUS_FALLBACK_REQUIRED, "this operation has no fixed kernel: the framework must run it");
  if (has_unbound_slot(op)) return refuse(e, NETRA_STATUS_BINDING, "a pointer argument of this operation was never bound");
  return launch_record(e, op, op.addresses, stream);
}

netra_status_t direct_launch(netra_engine* e, ProfileRecord& profile, cudaStream_t stream) {
  netra_status_t status = NETRA_STATUS_OK;
  for (size_t i = 0; i < profile.operations.size() && status == NETRA_STATUS_OK; ++i) status = launch_one(e, profile.operations[i], stream);
  return status;
}

// Code objects are shared between the engines of a process: engines built from the same cubin (two profiles of a model,
// or two engines bound to the two halves of a double-buffered serving loop) then run the same device code at the same
// addresses.  With a module per engine, alternating between two engines cost 10 us per 160 us decode step on a B200.
struct SharedModule {
  CUmodule module = nullptr;
  uint32_t users = 0;
};
std::mutex g_module_mutex;
std::map<std::tuple<int, size_t, size_t>, SharedModule> g_modules;      // (device, image size, image hash)

void release(netra_engine* e) {
  for (auto& p : e->profiles) {
    if (p.graph_exec) (void)cudaGraphExecDestroy(p.graph_exec);
    if (p.graph) (void)cudaGraphDestroy(p.graph);
  }
  if (driver().ok) {
    std::lock_guard<std::mutex> lock(g_module_mutex);
    for (auto& kv : e->modules) {
      if (!kv.second) continue;
      for (auto it = g_modules.begin(); it != g_modules.end(); ++it)
        if (it->second.module == kv.second) {
          if (--it->second.users == 0) {
            (void)driver().ModuleUnload(it->second.module);
            g_modules.erase(it);
          }
          break;
        }
    }
  }
  if (e->workspace) (void)cudaFree(e->workspace);
}

// ---- engine construction (throws CreateFailure) ------------------------------------------------------
void check_target(netra_engine* e, const Manifest& manifest) {
  int major = 0, warp = 0;
  (void)cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, e->device_id);
  (void)cudaDeviceGetAttribute(&warp, cudaDevAttrWarpSize, e->device_id);
  if (major != 10 || warp != 32) create_fail(NETRA_STATUS_UNSUPPORTED_TARGET, "device is not compute capability 10.x with 32-wide warps");
  int version = 0;
  const cudaError_t err = cudaDriverGetVersion(&version);
  if (err != cudaSuccess) create_fail(NETRA_STATUS_CUDA, std::string("cudaDriverGetVersion returned ") + cudaGetErrorString(err));
  const std::pair<uint32_t, uint32_t> have{(uint32_t)(version / 1000), (uint32_t)((version % 1000) / 10)};
  if (have < manifest.required_cuda)
    create_fail(NETRA_STATUS_UNSUPPORTED_TARGET, "the installed driver supports CUDA " + std::to_string(have.first) + "." + std::to_string(have.second) +
                                                     ", the engine requires " + std::to_string(manifest.required_cuda.first) + "." +
                                                     std::to_string(manifest.required_cuda.second));
}

CUmodule load_code_object(netra_engine* e, const std::string& relative) {
  CUmodule& module = e->modules[relative];
  if (module) return module;
  std::string image;
  try {
    image = read_file(e->directory + "/" + relative);
  } catch (const std::exception& ex) {
    create_fail(NETRA_STATUS_IO, ex.what());
  }
  std::lock_guard<std::mutex> lock(g_module_mutex);
  SharedModule& shared = g_modules[std::make_tuple(e->device_id, image.size(), std::hash<std::string>{}(image))];
  if (shared.module == nullptr) {
    const CUresult r = driver().ModuleLoadData(&shared.module, image.data());
    if (r != CUDA_SUCCESS) {
      g_modules.erase(std::make_tuple(e->device_id, image.size(), std::hash<std::string>{}(image)));
      create_fail(NETRA_STATUS_CUDA, "cuModuleLoadData(" + relative + ") returned CUresult " + std::to_string((int)r));
    }
  }
  ++shared.users;
  module = shared.module;
  return module;
}

void resolve_kernel(netra_engine* e, OpRecord& op) {
  const OpSpec& k = op.spec;
  CUresult r = driver().ModuleGetFunction(&op.function, load_code_object(e, k.cubin), k.symbol.c_str());
  if (r != CUDA_SUCCESS) create_fail(NETRA_STATUS_CUDA, "cuModuleGetFunction(" + k.symbol + ") returned CUresult " + std::to_string((int)r));
  if (k.dynamic_lds_bytes > 48 * 1024) {
    r = driver().FuncSetAttribute(op.function, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, (int)k.dynamic_lds_bytes);
    if (r != CUDA_SUCCESS) create_fail(NETRA_STATUS_CUDA, "cuFuncSetAttribute(" + k.symbol + ", dynamic shared memory) returned CUresult " + std::to_string((int)r));
  }
  if (k.registers_per_thread) {
    // kernels that move registers between warpgroups (setmaxnreg) only work for the allocation they were written for
    int regs = 0;
    r = driver().FuncGetAttribute(&regs, CU_FUNC_ATTRIBUTE_NUM_REGS, op.function);
    if (r != CUDA_SUCCESS) create_fail(NETRA_STATUS_CUDA, "cuFuncGetAttribute(" + k.symbol + ", registers) returned CUresult " + std::to_string((int)r));
    if ((uint32_t)regs != k.registers_per_thread)
      create_fail(NETRA_STATUS_MANIFEST, k.symbol + " was built with " + std::to_string(regs) + " registers per thread, the contract requires " +
                                             std::to_string(k.registers_per_thread));
  }
}

void wire_arguments(netra_engine* e, OpRecord& op) {
  op.argc = (uint32_t)op.spec.args.size();
  op.slots.reset(new ArgSlot[op.argc]);
  for (uint32_t i = 0; i < op.argc; ++i) {
    ArgSlot& slot = op.slots[i];
    slot.spec = op.spec.args[i];
    switch (slot.spec.kind) {
      case ArgSpec::U32:
        slot.scalar = slot.spec.value;
        op.addresses[i] = &slot.scalar;
        break;
      case ArgSpec::TensorMap:
      case ArgSpec::Pointer:
        if (!slot.spec.bindable && !slot.spec.null_pointer)
          slot.pointer = static_cast<unsigned char*>(e->workspace) + slot.spec.workspace_offset;
        if (slot.spec.kind == ArgSpec::TensorMap) {
          if (!slot.spec.bindable) {   // workspace tensor: the descriptor is final now; bound tensors get theirs in bind()
            if (!encode_map(&slot.map, slot.pointer, slot.spec.map))
              create_fail(NETRA_STATUS_CUDA, "cuTensorMapEncodeTiled refused the workspace tensor behind argument " + std::to_string(i) + " of " + op.spec.symbol);
            slot.map_ready = true;
          }
          op.addresses[i] = &slot.map;
        } else {
          op.addresses[i] = &slot.pointer;
        }
        break;
    }
  }
}

void build_engine(netra_engine* e) {
  (void)cudaFree(nullptr);   // make the primary context current for the driver entry points
  if (!driver().ok) create_fail(NETRA_STATUS_UNSUPPORTED_TARGET, "the CUDA driver does not export the entry points this runtime needs");
  Manifest manifest;
  try {
    manifest = parse_manifest(e->directory);
  } catch (const IoFailure& ex) {
    create_fail(NETRA_STATUS_IO, ex.what());
  } catch (const std::exception& ex) {
    create_fail(NETRA_STATUS_MANIFEST, ex.what());
  }
  check_target(e, manifest);
  e->workspace_bytes = manifest.workspace_bytes;
  if (e->workspace_bytes) {
    cudaError_t err = cudaMalloc(&e->workspace, (size_t)e->workspace_bytes);
    if (err != cudaSuccess) create_fail(NETRA_STATUS_CUDA, std::string("cudaMalloc(workspace) returned ") + cudaGetErrorString(err));
    err = cudaMemset(e->workspace, 0, (size_t)e->workspace_bytes);
    if (err != cudaSuccess) create_fail(NETRA_STATUS_CUDA, std::string("cudaMemset(workspace) returned ") + cudaGetErrorString(err));
  }
  e->profiles.resize(manifest.profiles.size());
  for (size_t p = 0; p < manifest.profiles.size(); ++p) {
    ProfileRecord& profile = e->profiles[p];
    profile.info = manifest.profiles[p].info;
    profile.operations.resize(manifest.operations.size());
    for (size_t o = 0; o < manifest.operations.size(); ++o) {
      OpRecord& op = profile.operations[o];
      op.spec = manifest.operations[o];
      if (op.spec.fallback) continue;
      resolve_kernel(e, op);
      wire_arguments(e, op);
    }
  }
}

}  // namespace

extern "C" netra_status_t netra_engine_check_manifest(const char* directory, char* error, size_t error_bytes) {
  if (!directory || !*directory) return NETRA_STATUS_INVALID_ARGUMENT;
  try {
    (void)parse_manifest(directory);
    if (error && error_bytes) error[0] = '\0';
    return NETRA_STATUS_OK;
  } catch (const std::exception& ex) {
    if (error && error_bytes) std::snprintf(error, error_bytes, "%s", ex.what());
    return NETRA_STATUS_MANIFEST;
  }
}

extern "C" const char* netra_engine_create_error(void) { return g_create_error.data(); }

extern "C" netra_status_t netra_engine_create(const char* directory, const netra_engine_options_t* options,
                                              netra_engine_t** output) {
  g_create_error[0] = '\0';
  if (!directory || !*directory || !options || !output || options->struct_size != sizeof(netra_engine_options_t))
    return NETRA_STATUS_INVALID_ARGUMENT;
  *output = nullptr;
  int caller_device = -1;
  if (cudaGetDevice(&caller_device) != cudaSuccess) {
    std::snprintf(g_create_error.data(), g_create_error.size(), "cudaGetDevice failed: no usable CUDA device");
    return NETRA_STATUS_CUDA;
  }
  if (cudaSetDevice(options->device_id) != cudaSuccess) {
    std::snprintf(g_create_error.data(), g_create_error.size(), "cudaSetDevice(%d) failed", (int)options->device_id);
    (void)cudaGetLastError();
    return NETRA_STATUS_CUDA;
  }
  std::unique_ptr<netra_engine> e(new (std::nothrow) netra_engine);
  netra_status_t status = NETRA_STATUS_OK;
  if (!e) {
    status = NETRA_STATUS_IO;
    std::snprintf(g_create_error.data(), g_create_error.size(), "out of host memory");
  } else {
    e->directory = directory;
    e->device_id = options->device_id;
    e->graph_enabled = options->enable_graph_capture != 0;
    try {
      build_engine(e.get());
    } catch (const CreateFailure& f) {
      status = f.status;
      std::snprintf(g_create_error.data(), g_create_error.size(), "%s", f.text.c_str());
    } catch (const std::exception& ex) {   // nothing may cross the C boundary
      status = NETRA_STATUS_MANIFEST;
      std::snprintf(g_create_error.data(), g_create_error.size(), "%s", ex.what());
    }
    if (status != NETRA_STATUS_OK) release(e.get());
  }
  (void)cudaSetDevice(caller_device);   // the caller's current device is restored on every path
  if (status != NETRA_STATUS_OK) return status;
  clear_error(e.get());
  *output = e.release();
  return NETRA_STATUS_OK;
}

extern "C" size_t netra_engine_profile_count(const netra_engine_t* e) { return e ? e->profiles.size() : 0; }

extern "C" netra_status_t netra_engine_query_profile(const netra_engine_t* e, uint32_t profile_id, netra_profile_info_t* output) {
  if (!e || !output || output->struct_size != sizeof(netra_profile_info_t)) return NETRA_STATUS_INVALID_ARGUMENT;
  if (profile_id >= e->profiles.size()) return NETRA_STATUS_UNSUPPORTED_PROFILE;
  *output = e->profiles[profile_id].info;
  return NETRA_STATUS_OK;
}

// ---- control plane: the caller serialises these -------------------------------------------------------
extern "C" netra_status_t netra_engine_bind(netra_engine_t* e, uint32_t profile_id, uint32_t operation_index,
                                            uint32_t argument_index, void* pointer) {
  if (!e || !pointer) return NETRA_STATUS_INVALID_ARGUMENT;
  // once the table is frozen (explicitly, by a captured graph, or while a launch reads it) it cannot change
  if (e->bindings_finalized.load(std::memory_order_acquire))
    return refuse(e, NETRA_STATUS_BUSY, "the binding table was frozen by finalize_bindings");
  if (e->in_flight.load(std::memory_order_acquire)) return refuse(e, NETRA_STATUS_BUSY, "a launch call is reading the binding table");
  if (profile_id >= e->profiles.size()) return refuse(e, NETRA_STATUS_BINDING, "no such profile");
  ProfileRecord& profile = e->profiles[profile_id];
  if (operation_index >= profile.operations.size()) return refuse(e, NETRA_STATUS_BINDING, "no such operation in this profile");
  if (profile.graph_prepared) return refuse(e, NETRA_STATUS_BUSY, "this profile's graph already holds the bound pointers");
  OpRecord& op = profile.operations[operation_index];
  if (argument_index >= op.argc) return refuse(e, NETRA_STATUS_BINDING, "no such argument in this operation");
  ArgSlot& slot = op.slots[argument_index];
  if (!slot.spec.bindable) return refuse(e, NETRA_STATUS_BINDING, "this argument is a constant or a workspace tensor, not a binding slot");
  if (slot.spec.kind == ArgSpec::TensorMap) {
    if ((reinterpret_cast<uintptr_t>(pointer) & 15u) != 0)
      return refuse(e, NETRA_STATUS_BINDING, "a tensor read through a TMA descriptor must start on a 16-byte boundary");
    if (!encode_map(&slot.map, pointer, slot.spec.map))
      return refuse(e, NETRA_STATUS_BINDING, "cuTensorMapEncodeTiled refused the pointer bound to this tensor-map slot");
    slot.map_ready = true;
  }
  slot.pointer = pointer;
  clear_error(e);
  return NETRA_STATUS_OK;
}

extern "C" netra_status_t netra_engine_finalize_bindings(netra_engine_t* e) {
  if (!e) return NETRA_STATUS_INVALID_ARGUMENT;
  if (e->in_flight.load(std::memory_order_acquire)) return refuse(e, NETRA_STATUS_BUSY, "a launch call is reading the binding table");
  for (const ProfileRecord& profile : e->profiles)
    for (const OpRecord& op : profile.operations)
      if (has_unbound_slot(op)) return refuse(e, NETRA_STATUS_BINDING, "every binding slot of every operation must be bound before the table is frozen");
  e->bindings_finalized.store(true, std::memory_order_release);
  clear_error(e);
  return NETRA_STATUS_OK;
}

extern "C" netra_status_t netra_engine_prepare_profile(netra_engine_t* e, uint32_t profile_id, cudaStream_t stream) {
  if (!e || profile_id >= e->profiles.size()) return NETRA_STATUS_INVALID_ARGUMENT;
  ProfileRecord& profile = e->profiles[profile_id];
  if (!e->graph_enabled || profile.graph_prepared) return NETRA_STATUS_OK;   // nothing to capture, or captured already
  if (profile.info.requires_fallback)
    return refuse(e, NETRA_STATUS_FALLBACK_REQUIRED, "a profile with a framework-fallback operation cannot be captured by this runtime");
  if (const netra_status_t frozen = netra_engine_finalize_bindings(e)) return frozen;
  cudaError_t err = cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal);
  if (err != cudaSuccess) return runtime_error(e, "cudaStreamBeginCapture", err);
  const netra_status_t enqueued = direct_launch(e, profile, stream);
  cudaGraph_t captured = nullptr;
  err = cudaStreamEndCapture(stream, &captured);   // always ends the capture, also after a refused launch
  if (enqueued != NETRA_STATUS_OK || err != cudaSuccess) {
    if (captured) (void)cudaGraphDestroy(captured);
    return enqueued != NETRA_STATUS_OK ? enqueued : runtime_error(e, "cudaStreamEndCapture", err);
  }
  err = cudaGraphInstantiate(&profile.graph_exec, captured, 0);
  if (err != cudaSuccess) {
    (void)cudaGraphDestroy(captured);
    return runtime_error(e, "cudaGraphInstantiate", err);
  }
  profile.graph = captured;
  profile.graph_prepared = true;
  return NETRA_STATUS_OK;
}

// ---- hot path: no allocation, no synchronisation, no file or string work ---------------------------------
extern "C" netra_status_t netra_engine_launch(netra_engine_t* e, uint32_t profile_id, const netra_launch_shape_t* shape,
                                              cudaStream_t stream) {
  LaunchContext ctx;
  if (const netra_status_t s = open_launch(e, profile_id, nullptr, shape, &ctx)) return s;
  ProfileRecord& profile = *ctx.profile;
  if (profile.info.requires_fallback)
    return refuse(e, NETRA_STATUS_FALLBACK_REQUIRED, "this profile contains an operation the framework must run");
  if (!profile.graph_prepared && !e->bindings_finalized.load(std::memory_order_acquire))
    return refuse(e, NETRA_STATUS_BINDING, "call finalize_bindings (or prepare_profile) before the first launch");
  InFlight guard(e);
  if (!profile.graph_prepared) return direct_launch(e, profile, stream);
  const cudaError_t err = cudaGraphLaunch(profile.graph_exec, stream);
  return err == cudaSuccess ? NETRA_STATUS_OK : runtime_error(e, "cudaGraphLaunch", err);
}

extern "C" netra_status_t netra_engine_launch_operation(netra_engine_t* e, uint32_t profile_id, uint32_t operation_index,
                                                        const netra_launch_shape_t* shape, cudaStream_t stream) {
  LaunchContext ctx;
  if (const netra_status_t s = open_launch(e, profile_id, &operation_index, shape, &ctx)) return s;
  if (ctx.profile->graph_prepared)
    return refuse(e, NETRA_STATUS_BUSY, "this profile runs as a captured graph: its operations can no longer be launched one by one");
  if (ctx.op->spec.fallback) return refuse(e, NETRA_STATUS_FALLBACK_REQUIRED, "this operation has no fixed kernel: the framework must run it");
  if (!e->bindings_finalized.load(std::memory_order_acquire))
    return refuse(e, NETRA_STATUS_BINDING, "call finalize_bindings before the first launch");
  InFlight guard(e);
  return launch_one(e, *ctx.op, stream);
}

extern "C" netra_status_t netra_engine_launch_operation_bound(netra_engine_t* e, uint32_t profile_id, uint32_t operation_index,
                                                              const netra_launch_shape_t* shape,
                                                              const netra_pointer_binding_t* bindings, uint32_t binding_count,
                                                              cudaStream_t stream) {
  if ((binding_count != 0 && bindings == nullptr) || binding_count > 16) return NETRA_STATUS_INVALID_ARGUMENT;
  LaunchContext ctx;
  if (const netra_status_t s = open_launch(e, profile_id, &operation_index, shape, &ctx)) return s;
  if (ctx.profile->graph_prepared)
    return refuse(e, NETRA_STATUS_BUSY, "this profile runs as a captured graph: per-call pointers cannot be supplied any more");
  OpRecord& op = *ctx.op;
  if (op.spec.fallback) return refuse(e, NETRA_STATUS_FALLBACK_REQUIRED, "this operation has no fixed kernel: the framework must run it");

  // The call must name each binding slot of the operation exactly once.  `seen` has one bit per argument.
  uint32_t seen = 0, slots = 0;
  for (uint32_t i = 0; i < op.argc; ++i) slots += op.slots[i].spec.bindable ? 1u : 0u;
  for (uint32_t i = 0; i < binding_count; ++i) {
    const netra_pointer_binding_t& b = bindings[i];
    if (b.reserved != 0 || b.pointer == nullptr || b.argument_index >= op.argc || !op.slots[b.argument_index].spec.bindable)
      return refuse(e, NETRA_STATUS_BINDING, "a per-call binding names no binding slot of this operation, or carries a null pointer");
    if (seen & (1u << b.argument_index)) return refuse(e, NETRA_STATUS_BINDING, "a binding slot appears twice in the per-call bindings");
    seen |= 1u << b.argument_index;
  }
  if (binding_count != slots) return refuse(e, NETRA_STATUS_BINDING, "the per-call bindings must cover every binding slot of the operation");

  // Argument storage private to this call, so that concurrent calls with different pointers cannot interfere.
  void* pointers[kMaxArguments];
  void* addresses[kMaxArguments];
  alignas(64) CUtensorMap maps[16];
  uint32_t maps_used = 0;
  for (uint32_t i = 0; i < op.argc; ++i) addresses[i] = op.addresses[i];
  for (uint32_t i = 0; i < binding_count; ++i) {
    const uint32_t arg = bindings[i].argument_index;
    if (op.slots[arg].spec.kind != ArgSpec::TensorMap) {
      pointers[arg] = bindings[i].pointer;
      addresses[arg] = &pointers[arg];
      continue;
    }
    const bool aligned = (reinterpret_cast<uintptr_t>(bindings[i].pointer) & 15u) == 0;
    if (!aligned || !encode_map(&maps[maps_used], bindings[i].pointer, op.slots[arg].spec.map))
      return refuse(e, NETRA_STATUS_BINDING, "cuTensorMapEncodeTiled refused a per-call pointer (tensor-map slots need 16-byte alignment)");
    addresses[arg] = &maps[maps_used++];
  }
  InFlight guard(e);
  return launch_record(e, op, addresses, stream);
}

extern "C" const char* netra_engine_last_error(const netra_engine_t* e) { return e ? e->last_error.data() : "netra_engine is null"; }

extern "C" void* netra_engine_workspace(const netra_engine_t* e) { return e ? e->workspace : nullptr; }

extern "C" netra_status_t netra_engine_destroy(netra_engine_t* e) {
  if (!e) return NETRA_STATUS_OK;
  if (e->in_flight.load(std::memory_order_acquire)) return refuse(e, NETRA_STATUS_BUSY, "a launch call is still inside the runtime");
  release(e);
  delete e;
  return NETRA_STATUS_OK;
}

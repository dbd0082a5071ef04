"""ctypes binding of the engine runtime ABI (``include/netra_engine.h``) plus a small session
helper that binds torch tensors by logical name using the engine's ``graph_recipe.json``.

The call order is the reference's (``runtime/gfx950/engine/README.md``): create -> query_profile ->
bind* -> finalize_bindings -> [prepare_profile] -> launch*, destroy.
"""
from __future__ import annotations

import ctypes
import json
from pathlib import Path
from typing import Mapping

from . import abi

STATUS = {0: "OK", 1: "INVALID_ARGUMENT", 2: "IO", 3: "MANIFEST", 4: "UNSUPPORTED_TARGET", 5: "UNSUPPORTED_PROFILE",
          6: "BINDING", 7: "CUDA", 8: "BUSY", 9: "FALLBACK_REQUIRED"}
c_void_p, c_u32, c_u64, c_i32 = ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_int32


class EngineOptions(ctypes.Structure):
    _fields_ = [("struct_size", c_u32), ("device_id", c_i32), ("enable_graph_capture", c_u32)]


class ProfileInfo(ctypes.Structure):
    _fields_ = [("struct_size", c_u32), ("profile_id", c_u32), ("min_m", c_u32), ("max_m", c_u32), ("min_batch", c_u32),
                ("max_batch", c_u32), ("min_sequence", c_u64), ("max_sequence", c_u64), ("tensor_parallel", c_u32),
                ("workspace_bytes", c_u64), ("requires_fallback", c_u32)]


class LaunchShape(ctypes.Structure):
    _fields_ = [("m", c_u32), ("batch", c_u32), ("sequence", c_u64), ("tensor_parallel", c_u32)]


class PointerBinding(ctypes.Structure):
    _fields_ = [("argument_index", c_u32), ("reserved", c_u32), ("pointer", c_void_p)]


ENGINE_SIGNATURES = {
    "netra_engine_create": (ctypes.c_int, [ctypes.c_char_p, ctypes.POINTER(EngineOptions), ctypes.POINTER(c_void_p)]),
    "netra_engine_profile_count": (ctypes.c_size_t, [c_void_p]),
    "netra_engine_query_profile": (ctypes.c_int, [c_void_p, c_u32, ctypes.POINTER(ProfileInfo)]),
    "netra_engine_bind": (ctypes.c_int, [c_void_p, c_u32, c_u32, c_u32, c_void_p]),
    "netra_engine_finalize_bindings": (ctypes.c_int, [c_void_p]),
    "netra_engine_prepare_profile": (ctypes.c_int, [c_void_p, c_u32, c_void_p]),
    "netra_engine_launch": (ctypes.c_int, [c_void_p, c_u32, ctypes.POINTER(LaunchShape), c_void_p]),
    "netra_engine_launch_operation": (ctypes.c_int, [c_void_p, c_u32, c_u32, ctypes.POINTER(LaunchShape), c_void_p]),
    "netra_engine_launch_operation_bound": (ctypes.c_int, [c_void_p, c_u32, c_u32, ctypes.POINTER(LaunchShape),
                                                           ctypes.POINTER(PointerBinding), c_u32, c_void_p]),
    "netra_engine_last_error": (ctypes.c_char_p, [c_void_p]),
    "netra_engine_destroy": (ctypes.c_int, [c_void_p]),
    "netra_engine_check_manifest": (ctypes.c_int, [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_size_t]),
    "netra_engine_workspace": (c_void_p, [c_void_p]),
    "netra_engine_create_error": (ctypes.c_char_p, []),
}

_typed = False


def load() -> ctypes.CDLL:
    global _typed
    lib = abi.load()
    if not _typed:
        for name, (restype, argtypes) in ENGINE_SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = restype, argtypes
        _typed = True
    return lib


class EngineError(RuntimeError):
    def __init__(self, status: int, what: str, message: str = ""):
        super().__init__(f"{what}: NETRA_STATUS_{STATUS.get(status, status)}" + (f" ({message})" if message else ""))
        self.status = status


def check_manifest(directory: Path | str) -> tuple[int, str]:
    buf = ctypes.create_string_buffer(512)
    rc = load().netra_engine_check_manifest(str(directory).encode(), buf, len(buf))
    return rc, buf.value.decode(errors="replace")


class EngineSession:
    """One loaded engine with tensors bound by logical name."""

    def __init__(self, directory: Path | str, device_id: int = 0, enable_graph_capture: bool = True):
        self.lib = load()
        self.directory = Path(directory)
        self.recipe = json.loads((self.directory / "graph_recipe.json").read_text())
        self.manifest = json.loads((self.directory / "engine.json").read_text())
        self.layout_plan = json.loads((self.directory / "layout_plan.json").read_text())
        options = EngineOptions(ctypes.sizeof(EngineOptions), device_id, int(enable_graph_capture))
        handle = c_void_p()
        rc = self.lib.netra_engine_create(str(self.directory).encode(), ctypes.byref(options), ctypes.byref(handle))
        if rc != 0:
            raise EngineError(rc, "netra_engine_create", self.lib.netra_engine_create_error().decode(errors="replace"))
        self.handle = handle
        self._keep = []
        guards = self.manifest["profiles"][0]["guards"]
        self.shape = LaunchShape(guards["m"]["min"], max(1, guards["batch"]["min"]), guards["sequence"]["min"],
                                 self.manifest["profiles"][0]["tensor_parallel"])

    def _check(self, rc: int, what: str) -> None:
        if rc != 0:
            raise EngineError(rc, what, self.lib.netra_engine_last_error(self.handle).decode(errors="replace"))

    def profile(self, profile_id: int = 0) -> ProfileInfo:
        info = ProfileInfo()
        info.struct_size = ctypes.sizeof(info)
        self._check(self.lib.netra_engine_query_profile(self.handle, profile_id, ctypes.byref(info)), "query_profile")
        return info

    def prepare_weights(self, tensors: Mapping[str, "object"]) -> dict:
        """Applies the engine's layout plan (weight repack) and returns the tensors to bind."""
        import torch
        out = dict(tensors)
        for step in self.layout_plan.get("steps", []):
            if step["entry_point"] == "netra_moe_mxfp4_pack_launch":     # codes and scale bytes are re-ordered together
                from .moe import pack_mxfp4
                out[step["tensor"]], out[step["scale_tensor"]] = pack_mxfp4(out[step["tensor"]], out[step["scale_tensor"]],
                                                                            paired_half_rows=int(step["paired_half_rows"]))
                continue
            w = out[step["tensor"]]
            packed = torch.empty_like(w)
            abi.check(self.lib.netra_moe_repack_tiles_launch(packed.data_ptr(), w.data_ptr(), w.shape[0] * w.shape[1],
                                                             w.shape[2] * w.element_size(),
                                                             torch.cuda.current_stream().cuda_stream), "repack_tiles_launch")
            out[step["tensor"]] = packed
        return out

    def bind(self, tensors: Mapping[str, "object"], profile_id: int = 0) -> None:
        slots = self.recipe["binding_slots"]
        missing = sorted(set(slots) - set(tensors))
        if missing:
            raise KeyError(f"tensors not provided for binding: {missing}")
        for name, places in slots.items():
            t = tensors[name]
            self._keep.append(t)
            for place in places:
                self._check(self.lib.netra_engine_bind(self.handle, profile_id, place["operation"], place["argument"],
                                                       t.data_ptr()), f"bind {name}")

    def finalize(self) -> None:
        self._check(self.lib.netra_engine_finalize_bindings(self.handle), "finalize_bindings")

    def prepare(self, stream: int, profile_id: int = 0) -> None:
        self._check(self.lib.netra_engine_prepare_profile(self.handle, profile_id, stream), "prepare_profile")

    def launch(self, stream: int, profile_id: int = 0, shape: LaunchShape | None = None) -> None:
        self._check(self.lib.netra_engine_launch(self.handle, profile_id, ctypes.byref(shape or self.shape), stream), "launch")

    def launch_operation(self, index: int, stream: int, profile_id: int = 0) -> None:
        self._check(self.lib.netra_engine_launch_operation(self.handle, profile_id, index, ctypes.byref(self.shape), stream),
                    "launch_operation")

    def workspace_view(self, name: str, dtype, device):
        """torch view of one workspace tensor (engine-owned memory)."""
        import torch
        entry = self.recipe["workspace_tensors"][name]
        base = self.lib.netra_engine_workspace(self.handle)
        nbytes = entry["bytes"]
        holder = _DevicePointer(base + entry["offset"], nbytes)
        return torch.as_tensor(holder, device=device).view(dtype)

    def close(self) -> None:
        if getattr(self, "handle", None):
            rc = self.lib.netra_engine_destroy(self.handle)
            if rc == 0:
                self.handle = None
            return rc
        return 0

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class _DevicePointer:
    """Minimal ``__cuda_array_interface__`` holder for a raw device range (uint8)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}

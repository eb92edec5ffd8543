"""Runs a compiled plan's generated kernels on the CPU: the CUDA source the plan compiler emits is compiled with g++
against a small shim of the CUDA execution model (one OS thread per CUDA thread of a block, see shim.h) and the plan's
kernel steps are executed in order over NumPy buffers. Test infrastructure for the generated code (pointwise, reduction,
row, window, sort, random-bit, factorization and attention kernels); plans with steps that are hand-written CUDA
(contractions, the built-in scatter) or control flow are reported as unsupported. Nothing in the product imports this."""
from __future__ import annotations

import ctypes as C
import hashlib
import os
import re
import subprocess
import tempfile
from pathlib import Path

import numpy as np

import b200

HERE = Path(__file__).resolve().parent
_NP = {"f32": np.float32, "f64": np.float64, "i8": np.int8, "i16": np.int16, "i32": np.int32, "i64": np.int64,
       "ui8": np.uint8, "ui16": np.uint16, "ui32": np.uint32, "ui64": np.uint64, "i1": np.bool_, "bf16": np.uint16,
       "f16": np.float16}


class Unsupported(Exception):
    pass


_HOST_CONVERSIONS = '''
DEV void pdl_prologue() {}
DEV float bf16_to_f(u16 h) { return __uint_as_float(((u32)h) << 16); }
DEV u16 f_to_bf16(float f) {
  u32 u = __float_as_uint(f);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (u16)0x7FFF;
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (u16)(u >> 16);
}
DEV float f16_to_f(u16 h) { _Float16 v; std::memcpy(&v, &h, 2); return (float)v; }
DEV u16 f_to_f16(float f) { _Float16 v = (_Float16)f; u16 h; std::memcpy(&h, &v, 2); return h; }
'''


def _host_source(src: str) -> str:
    """The generated translation unit with its four inline-PTX helpers replaced by C++."""
    out, skip = [], False
    for line in src.splitlines():
        if re.match(r"DEV (void pdl_prologue|float bf16_to_f|u16 f_to_bf16|float f16_to_f|u16 f_to_f16)\(", line):
            if "{" in line and line.rstrip().endswith("}"):
                continue                                    # one-line definition
            skip = True
            continue
        if skip:
            if line.startswith("}"):
                skip = False
            continue
        out.append(line)
    text = "\n".join(out)
    at = text.index("#define DEV")
    at = text.index("\n", at) + 1
    return '#include "shim.h"\n' + text[:at] + _HOST_CONVERSIONS + text[at:]


def _cache_dir() -> Path:
    d = Path(tempfile.gettempdir()) / "b200_cuda_emu"
    d.mkdir(exist_ok=True)
    return d


def _compile(cmd, what):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"g++ failed on {what}:\n" + r.stderr[:6000])


def _runner() -> Path:
    """The thread team and its barriers, built once."""
    key = hashlib.sha256(((HERE / "shim.h").read_text() + (HERE / "runner.cc").read_text()).encode()).hexdigest()[:24]
    so = _cache_dir() / f"libemu_runner_{key}.so"
    if not so.exists():
        _compile(["g++", "-std=c++17", "-O1", "-g0", "-w", "-fPIC", "-shared", "-pthread", f"-I{HERE}", str(HERE / "runner.cc"), "-o", str(so) + ".tmp"],
                 "the runner")
        os.replace(str(so) + ".tmp", so)
    return so


def _build(src: str):
    runner = _runner()
    host = _host_source(src)
    key = hashlib.sha256((host + runner.name).encode()).hexdigest()[:24]
    so = _cache_dir() / f"k{key}.so"
    if not so.exists():
        cu = _cache_dir() / f"k{key}.cc"
        cu.write_text(host)
        _compile(["g++", "-std=c++17", "-O0", "-g0", "-w", "-fPIC", "-shared", f"-I{HERE}", str(cu), str(runner), f"-Wl,-rpath,{runner.parent}",
                  "-o", str(so) + ".tmp"], "the generated source")
        os.replace(str(so) + ".tmp", so)
    return C.CDLL(str(runner), mode=C.RTLD_GLOBAL), C.CDLL(str(so))


def _aligned(nbytes: int) -> np.ndarray:
    raw = np.zeros(max(nbytes, 1) + 256, np.uint8)
    off = (-raw.ctypes.data) % 256
    return raw[off:off + max(nbytes, 1)]


def _to_bf16_bits(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return np.where(nan, np.uint16(0x7FFF), r)


def _scatter_elems(slots, numel, updates, computation, nbytes, args):
    """The hand-written part of a general scatter, restated: the operand becomes the result, the (destination, update)
    pairs the generated key kernel left in the scratch are sorted by destination, ties in update order (the device
    does it by radix passes that end in either half of the scratch: both halves get the sorted pairs here), and a
    built-in update computation (0 assign, 1 add, 2 multiply, 3 minimum, 4 maximum) is folded into the result in that
    order; a computation of its own (-1) is left to the generated kernel that follows."""
    operand, _, upd, out, scratch = (slots[a] for a in args)
    out[0][:nbytes] = operand[0][:nbytes]
    sc = scratch[0][:scratch[0].size // 4 * 4].view(np.int32)
    key, order = sc[:updates].copy(), sc[updates:2 * updates].copy()
    perm = np.argsort(key, kind="stable")
    for base in (0, 2 * updates):
        sc[base:base + updates] = key[perm]
        sc[base + updates:base + 2 * updates] = order[perm]
    if computation < 0:
        return
    dt = out[2]
    view = lambda s: s[0][:s[0].size // np.dtype(_NP[s[2]]).itemsize * np.dtype(_NP[s[2]]).itemsize].view(_NP[s[2]])
    o, u = view(out), view(upd)
    if dt == "bf16":
        raise Unsupported("built-in scatter on bf16")
    fold = {0: lambda a, v: v, 1: lambda a, v: a + v, 2: lambda a, v: a * v,
            3: lambda a, v: v if (v < a or v != v) else a, 4: lambda a, v: v if (v > a or v != v) else a}[computation]
    with np.errstate(all="ignore"):
        for k, q in zip(key[perm], order[perm]):
            if k < numel:
                o[k] = fold(o[k], u[q])


def run_plan_on_cpu(text: str, inputs: list) -> list:
    """Compiles `text`, runs the plan's kernel steps on host threads and returns the results as NumPy arrays (bf16
    results as float32)."""
    plan, src = b200.compile_to_plan(text, slots=True)
    _, table = plan.split("slots:\n")
    table, launches = table.split("launches:\n")
    steps = []
    for line in launches.splitlines():
        m = re.match(r"^  kernel (\S+) grid=(\d+)x(\d+)x(\d+) block=(\d+)x(\d+)x(\d+) args=\[([\d,]*)\]\s*$", line)
        if m:
            steps.append(("kernel", m.group(1), [int(m.group(k)) for k in range(2, 8)], [int(v) for v in m.group(8).split(",") if v]))
            continue
        m = re.match(r"^  memcpy bytes=(\d+) args=\[(\d+),(\d+)\]\s*$", line)
        if m:
            steps.append(("memcpy", int(m.group(1)), None, [int(m.group(2)), int(m.group(3))]))
            continue
        m = re.match(r"^  scatter_elems numel=(\d+) updates=(\d+) computation=(-?\d+) bytes=(\d+) args=\[([\d,]*)\]\s*$", line)
        if m:
            steps.append(("scatter", [int(m.group(k)) for k in range(1, 5)], None, [int(v) for v in m.group(5).split(",") if v]))
            continue
        raise Unsupported(line.strip()[:80])
    slots, results = {}, {}
    for line in table.splitlines():
        m = re.match(r"^  slot (\d+) (\w+) index=(-?\d+) arena=\d+ offset=\d+ bytes=(\d+) (\S+)(?: hex=(\S*))?$", line)
        if m:
            sid, kind, index, nbytes, ty, hx = int(m.group(1)), m.group(2), int(m.group(3)), int(m.group(4)), m.group(5), m.group(6)
            buf = _aligned(nbytes)
            tm = re.match(r"tensor<((?:\d+x)*)(\w+)>", ty)
            shape = tuple(int(v) for v in tm.group(1).split("x") if v) if tm else ()
            dt = tm.group(2) if tm else "ui8"
            if kind == "arg":
                a = np.asarray(inputs[index])
                raw = _to_bf16_bits(a) if dt == "bf16" else np.ascontiguousarray(a, _NP[dt])
                buf[:raw.nbytes] = raw.reshape(-1).view(np.uint8)
            elif kind == "const":
                if hx in (None, "-"):
                    raise Unsupported("constant without data")
                data = np.frombuffer(bytes.fromhex(hx), np.uint8)
                buf[:data.size] = data
            slots[sid] = (buf, shape, dt)
            continue
        m = re.match(r"^  result (\d+) slot=(\d+) tensor<((?:\d+x)*)(\w+)>$", line)
        if m:                            # a result may be a reshaped view of a slot: its own type counts
            results[int(m.group(1))] = (int(m.group(2)), tuple(int(v) for v in m.group(3).split("x") if v), m.group(4))
    runner, lib = _build(src)
    runner.emu_launch.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]
    runner.emu_launch.restype = None
    for kind, name, dims, args in steps:
        if kind == "memcpy":
            slots[args[0]][0][:name] = slots[args[1]][0][:name]
            continue
        if kind == "scatter":
            _scatter_elems(slots, *name, args)
            continue
        fn = C.cast(getattr(lib, name), C.c_void_p)
        ptrs = (C.c_void_p * len(args))(*[slots[a][0].ctypes.data for a in args])
        runner.emu_launch(fn, len(args), ptrs, *dims)
    outs = []
    for k in sorted(results):
        sid, shape, dt = results[k]
        buf = slots[sid][0]
        n = int(np.prod(shape, dtype=np.int64)) if shape else 1
        a = buf[:n * np.dtype(_NP[dt]).itemsize].view(_NP[dt]).reshape(shape).copy()
        if dt == "bf16":
            a = (a.astype(np.uint32) << 16).view(np.float32)
        outs.append(a)
    return outs

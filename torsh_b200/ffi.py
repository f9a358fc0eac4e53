"""Foreign-language surface built on the C ABI (``crates/torsh-ffi/src``): header parser and unified type table
(``type_system.rs``, ``conversions.rs``), binding generators for Python ctypes, C#, Go, Java, Julia, Lua, MATLAB, Node.js
(+ TypeScript), R, Ruby, Swift and WebAssembly glue (``binding_generator.rs``, ``csharp.rs``, ``go.rs``, ``java.rs``,
``julia.rs``, ``lua.rs``, ``matlab.rs``, ``nodejs/``, ``r_lang.rs``, ``ruby.rs``, ``swift.rs``, ``wasm.rs``), API
reference and test generation (``api_docs.rs``, ``test_generator.rs``), status-to-exception mapping (``error.rs``), call
batching (``performance.rs``), NumPy protocol support (``numpy_compatibility.rs``), pandas and SciPy bridges
(``pandas_support.rs``, ``scipy_integration.rs``), SVG / text plots and notebook HTML views (``plotting_utilities.rs``,
``jupyter_widgets.rs``) and source migration from other frameworks (``migration_tools.rs``)."""
from __future__ import annotations

import ast
import html
import math
import re
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Sequence

import numpy as np
import torch

HEADER = Path(__file__).resolve().parent.parent / "csrc" / "include" / "torsh.h"
STATUS_NAMES = {0: "ok", 1: "invalid argument", 2: "shape mismatch", 3: "out of memory", 4: "not available"}


class TorshFfiError(RuntimeError):
    def __init__(self, status: int, detail: str = ""):
        super().__init__(f"{STATUS_NAMES.get(status, 'error')} (status {status})" + (f": {detail}" if detail else ""))
        self.status = status


# ================================================================================================ header model
@dataclass
class CParam:
    ctype: str
    name: str


@dataclass
class CFunction:
    name: str
    ret: str
    params: list
    doc: str = ""

    @property
    def group(self): return self.name.split("_")[1] if self.name.count("_") > 1 and self.name.split("_")[1] in ("tensor", "linear", "optimizer", "sgd", "adam", "cuda", "module") else "runtime"
    def signature(self): return f"{self.ret} {self.name}({', '.join(f'{p.ctype} {p.name}' for p in self.params) or 'void'})"


def _norm_type(t: str) -> str:
    t = re.sub(r"\s+", " ", t.strip())
    return re.sub(r"\s*\*", "*", t)


def parse_header(text: str | None = None) -> list[CFunction]:
    """Function declarations of a C header (comments kept as documentation of the declaration that follows them)."""
    text = HEADER.read_text() if text is None else text
    out, pending_doc = [], ""
    body = re.sub(r"#[^\n]*", "", text)
    body = re.sub(r"typedef[^;]*;[ \t]*(/\*.*?\*/)?", "", body)
    for m in re.finditer(r"/\*(.*?)\*/|([A-Za-z_][\w\s\*]*?\b(\w+)\s*\(([^;{}()]*)\)\s*;)([ \t]*/\*(.*?)\*/)?", body, re.S):
        if m.group(1) is not None:
            pending_doc, doc_end = " ".join(m.group(1).split()), m.end(); continue
        decl, name, params = m.group(2), m.group(3), m.group(4)
        if pending_doc and body[doc_end:m.start(2)].count("\n") > 1:                # a comment separated by a blank line is not this declaration's
            pending_doc = ""
        if decl.lstrip().startswith("typedef"):
            pending_doc = ""; continue
        ret = _norm_type(decl[:decl.index(name)])
        ps = []
        if params.strip() and params.strip() != "void":
            for i, p in enumerate(params.split(",")):
                p = " ".join(p.split())
                mm = re.match(r"(.*?)(\w+)$", p)
                ps.append(CParam(_norm_type(mm.group(1)), mm.group(2)) if mm and mm.group(1).strip() else CParam(_norm_type(p), f"arg{i}"))
        trailing = " ".join((m.group(6) or "").split())
        out.append(CFunction(name, ret, ps, trailing or pending_doc)); pending_doc = ""
    return out


_HANDLES = ("TorshTensor", "TorshLinear", "TorshOptimizer", "TorshModule")
# canonical kind -> type in each language
TYPE_TABLE = {
    "void":    {"python": "None", "csharp": "void", "go": "", "java": "void", "julia": "Cvoid", "lua": "void", "node": "'void'", "ts": "void", "ruby": ":void", "swift": "Void", "r": "NULL", "matlab": "void"},
    "int":     {"python": "ctypes.c_int", "csharp": "int", "go": "C.int", "java": "int", "julia": "Cint", "lua": "int", "node": "'int'", "ts": "number", "ruby": ":int", "swift": "Int32", "r": "integer", "matlab": "int32"},
    "bool":    {"python": "ctypes.c_bool", "csharp": "[MarshalAs(UnmanagedType.I1)] bool", "go": "C.bool", "java": "boolean", "julia": "Bool", "lua": "bool", "node": "'bool'", "ts": "boolean", "ruby": ":bool", "swift": "Bool", "r": "logical", "matlab": "logical"},
    "int64":   {"python": "ctypes.c_int64", "csharp": "long", "go": "C.int64_t", "java": "long", "julia": "Int64", "lua": "int64_t", "node": "'int64'", "ts": "bigint", "ruby": ":int64", "swift": "Int64", "r": "numeric", "matlab": "int64"},
    "uint64":  {"python": "ctypes.c_uint64", "csharp": "ulong", "go": "C.uint64_t", "java": "long", "julia": "UInt64", "lua": "uint64_t", "node": "'uint64'", "ts": "bigint", "ruby": ":uint64", "swift": "UInt64", "r": "numeric", "matlab": "uint64"},
    "size":    {"python": "ctypes.c_size_t", "csharp": "UIntPtr", "go": "C.size_t", "java": "long", "julia": "Csize_t", "lua": "size_t", "node": "'size_t'", "ts": "number", "ruby": ":size_t", "swift": "Int", "r": "numeric", "matlab": "uint64"},
    "float":   {"python": "ctypes.c_float", "csharp": "float", "go": "C.float", "java": "float", "julia": "Cfloat", "lua": "float", "node": "'float'", "ts": "number", "ruby": ":float", "swift": "Float", "r": "numeric", "matlab": "single"},
    "double":  {"python": "ctypes.c_double", "csharp": "double", "go": "C.double", "java": "double", "julia": "Cdouble", "lua": "double", "node": "'double'", "ts": "number", "ruby": ":double", "swift": "Double", "r": "numeric", "matlab": "double"},
    "string":  {"python": "ctypes.c_char_p", "csharp": "IntPtr", "go": "*C.char", "java": "String", "julia": "Cstring", "lua": "const char*", "node": "'str'", "ts": "string", "ruby": ":string", "swift": "UnsafePointer<CChar>?", "r": "character", "matlab": "cstring"},
    "floatptr": {"python": "ctypes.POINTER(ctypes.c_float)", "csharp": "float[]", "go": "*C.float", "java": "float[]", "julia": "Ptr{Cfloat}", "lua": "float*", "node": "'float*'", "ts": "Float32Array", "ruby": ":pointer", "swift": "UnsafeMutablePointer<Float>?", "r": "numeric", "matlab": "singlePtr"},
    "int64ptr": {"python": "ctypes.POINTER(ctypes.c_int64)", "csharp": "long[]", "go": "*C.int64_t", "java": "long[]", "julia": "Ptr{Int64}", "lua": "int64_t*", "node": "'int64*'", "ts": "BigInt64Array", "ruby": ":pointer", "swift": "UnsafeMutablePointer<Int64>?", "r": "numeric", "matlab": "int64Ptr"},
    "handle":  {"python": "ctypes.c_void_p", "csharp": "IntPtr", "go": "unsafe.Pointer", "java": "long", "julia": "Ptr{Cvoid}", "lua": "void*", "node": "'void*'", "ts": "unknown", "ruby": ":pointer", "swift": "OpaquePointer?", "r": "externalptr", "matlab": "voidPtr"},
}


def canonical(ctype: str) -> str:
    t = ctype.replace("const ", "").strip()
    if t.endswith("*"):
        base = t[:-1].strip()
        return "handle" if base in _HANDLES or base == "void" else "string" if base == "char" else "floatptr" if base == "float" else "int64ptr" if base == "int64_t" else "handle"
    return {"void": "void", "int": "int", "TorshStatus": "int", "bool": "bool", "int64_t": "int64", "uint64_t": "uint64", "size_t": "size", "float": "float", "double": "double"}[t]


def lang_type(ctype: str, lang: str) -> str: return TYPE_TABLE[canonical(ctype)][lang]
def _camel(name: str) -> str: return "".join(p.capitalize() for p in name.removeprefix("torsh_").split("_"))


# ================================================================================================ generators
class BindingGenerator:
    def __init__(self, functions: Sequence[CFunction] | None = None, library: str = "torsh_b200_host"): self.fns, self.lib = list(functions or parse_header()), library
    LANGUAGES = ("python", "csharp", "go", "java", "julia", "lua", "matlab", "nodejs", "typescript", "r", "ruby", "swift", "wasm")
    def generate(self, lang: str) -> str: return getattr(self, lang)()
    def generate_all(self, out_dir) -> dict:
        out_dir, ext = Path(out_dir), {"python": "torsh_ffi.py", "csharp": "Torsh.cs", "go": "torsh.go", "java": "Torsh.java", "julia": "Torsh.jl", "lua": "torsh.lua", "matlab": "torsh_proto.m", "nodejs": "torsh.js",
                                       "typescript": "torsh.d.ts", "r": "torsh.R", "ruby": "torsh.rb", "swift": "Torsh.swift", "wasm": "torsh_wasm.js"}
        out_dir.mkdir(parents=True, exist_ok=True)
        files = {}
        for lang in self.LANGUAGES:
            (out_dir / ext[lang]).write_text(self.generate(lang)); files[lang] = out_dir / ext[lang]
        return files

    def python(self) -> str:
        L = ['"""ctypes binding generated from the C header: argument and result types declared, status codes raised as exceptions."""', "import ctypes", "", "",
             "class TorshError(RuntimeError):", "    pass", "", "", "def load(path):", "    lib = ctypes.CDLL(path)"]
        for f in self.fns:
            L.append(f"    lib.{f.name}.restype = {lang_type(f.ret, 'python')}")
            L.append(f"    lib.{f.name}.argtypes = [{', '.join(lang_type(p.ctype, 'python') for p in f.params)}]")
        L += ["    return _Api(lib)", "", "", "class _Api:", "    def __init__(self, lib):", "        self.lib = lib", "",
              "    def _check(self, status):", "        if status != 0:", "            raise TorshError(f\"status {status}: {(self.lib.torsh_get_last_error() or b'').decode()}\")", "",
              "    def _handle(self, h, what):", "        if not h:", "            raise TorshError(f\"{what} failed: {(self.lib.torsh_get_last_error() or b'').decode()}\")", "        return ctypes.c_void_p(h)", ""]
        for f in self.fns:
            names = [p.name for p in f.params]
            call = f"self.lib.{f.name}({', '.join(names)})"
            body = f"self._check({call})" if f.ret == "TorshStatus" else f"return self._handle({call}, '{f.name}')" if canonical(f.ret) == "handle" else f"return {call}"
            doc = f'        """{f.signature()}' + (f" - {f.doc}" if f.doc else "") + '"""'
            L += [f"    def {f.name.removeprefix('torsh_')}({', '.join(['self'] + names)}):", doc, f"        {body}", ""]
        return "\n".join(L)

    def csharp(self) -> str:
        L = ["using System;", "using System.Runtime.InteropServices;", "", "namespace Torsh", "{", "    public static class Native", "    {", f'        const string Lib = "{self.lib}";']
        for f in self.fns:
            ps = ", ".join(f"{lang_type(p.ctype, 'csharp')} {p.name}" for p in f.params)
            L += [f'        [DllImport(Lib, CallingConvention = CallingConvention.Cdecl, EntryPoint = "{f.name}")]', f"        public static extern {lang_type(f.ret, 'csharp').replace('[MarshalAs(UnmanagedType.I1)] ', '')} {_camel(f.name)}({ps});"]
        L += ["    }", "", "    public sealed class Tensor : IDisposable", "    {", "        internal IntPtr Handle;", "        internal Tensor(IntPtr h) { if (h == IntPtr.Zero) throw new InvalidOperationException(Marshal.PtrToStringAnsi(Native.GetLastError())); Handle = h; }",
              "        public static Tensor FromArray(float[] data, long[] shape) => new Tensor(Native.TensorNew(data, shape, shape.Length));",
              "        public static Tensor operator +(Tensor a, Tensor b) => new Tensor(Native.TensorAdd(a.Handle, b.Handle));", "        public static Tensor operator *(Tensor a, Tensor b) => new Tensor(Native.TensorMul(a.Handle, b.Handle));",
              "        public Tensor MatMul(Tensor o) => new Tensor(Native.TensorMatmul(Handle, o.Handle));", "        public void Dispose() { if (Handle != IntPtr.Zero) { Native.TensorFree(Handle); Handle = IntPtr.Zero; } }", "    }", "}"]
        return "\n".join(L) + "\n"

    def go(self) -> str:
        L = ["package torsh", "", "/*", f"#cgo LDFLAGS: -l{self.lib}", '#include "torsh.h"', "#include <stdlib.h>", "*/", 'import "C"', "", 'import (', '\t"errors"', '\t"unsafe"', ")", "", "var _ = unsafe.Pointer(nil)", "",
             "func lastError() error { return errors.New(C.GoString(C.torsh_get_last_error())) }", ""]
        for f in self.fns:
            ps = ", ".join(f"{p.name} {self._go_t(p.ctype)}" for p in f.params)
            args = ", ".join(self._go_arg(p) for p in f.params)
            rt = self._go_t(f.ret)
            if f.ret == "TorshStatus":
                L += [f"func {_camel(f.name)}({ps}) error {{", f"\tif C.{f.name}({args}) != 0 {{", "\t\treturn lastError()", "\t}", "\treturn nil", "}", ""]
            elif f.ret == "void":
                L += [f"func {_camel(f.name)}({ps}) {{ C.{f.name}({args}) }}", ""]
            else:
                L += [f"func {_camel(f.name)}({ps}) {rt} {{ return {self._go_ret(f.ret, f'C.{f.name}({args})')} }}", ""]
        return "\n".join(L)

    @staticmethod
    def _go_t(c):
        k = canonical(c)
        base = c.replace("const ", "").rstrip("*").strip()
        return {"handle": f"*C.{base}" if base in _HANDLES else "unsafe.Pointer", "int": "int", "bool": "bool", "int64": "int64", "uint64": "uint64", "size": "uint64", "float": "float32", "double": "float64", "string": "string",
                "floatptr": "*float32", "int64ptr": "*int64", "void": ""}[k]
    @staticmethod
    def _go_arg(p):
        k = canonical(p.ctype)
        return {"int": f"C.int({p.name})", "bool": f"C.bool({p.name})", "int64": f"C.int64_t({p.name})", "uint64": f"C.uint64_t({p.name})", "size": f"C.size_t({p.name})", "float": f"C.float({p.name})", "double": f"C.double({p.name})",
                "floatptr": f"(*C.float)(unsafe.Pointer({p.name}))", "int64ptr": f"(*C.int64_t)(unsafe.Pointer({p.name}))", "string": f"C.CString({p.name})"}.get(k, p.name)
    @staticmethod
    def _go_ret(c, expr):
        k = canonical(c)
        return {"int": f"int({expr})", "bool": f"bool({expr})", "int64": f"int64({expr})", "uint64": f"uint64({expr})", "size": f"uint64({expr})", "float": f"float32({expr})", "double": f"float64({expr})", "string": f"C.GoString({expr})",
                "floatptr": f"(*float32)(unsafe.Pointer({expr}))"}.get(k, expr)

    def java(self) -> str:
        L = ["package org.torsh;", "", "/** JNI surface: one native method per C function; handles travel as long. */", "public final class Torsh {", f'    static {{ System.loadLibrary("{self.lib}_jni"); }}', "    private Torsh() {}"]
        for f in self.fns:
            L.append(f"    public static native {lang_type(f.ret, 'java')} {self._lower_camel(f.name)}({', '.join(lang_type(p.ctype, 'java') + ' ' + p.name for p in f.params)});")
        L += ["", "    public static final class Tensor implements AutoCloseable {", "        final long handle;", "        Tensor(long h) { if (h == 0) throw new IllegalStateException(getLastError()); handle = h; }",
              "        public static Tensor of(float[] data, long[] shape) { return new Tensor(tensorNew(data, shape, shape.length)); }", "        public Tensor add(Tensor o) { return new Tensor(tensorAdd(handle, o.handle)); }",
              "        public Tensor matmul(Tensor o) { return new Tensor(tensorMatmul(handle, o.handle)); }", "        @Override public void close() { tensorFree(handle); }", "    }", "}"]
        return "\n".join(L) + "\n"

    def jni_stubs(self) -> str:
        """C side of the Java class (compiled against ``jni.h`` into ``lib<name>_jni``)."""
        jt = {"void": "void", "int": "jint", "bool": "jboolean", "int64": "jlong", "uint64": "jlong", "size": "jlong", "float": "jfloat", "double": "jdouble", "string": "jstring", "floatptr": "jfloatArray", "int64ptr": "jlongArray", "handle": "jlong"}
        L = ["#include <jni.h>", '#include "torsh.h"', ""]
        for f in self.fns:
            ps = "".join(f", {jt[canonical(p.ctype)]} {p.name}" for p in f.params)
            pre, post, args = [], [], []
            for p in f.params:
                k = canonical(p.ctype)
                if k == "floatptr":
                    pre.append(f"  jfloat* {p.name}_p = {p.name} ? (*env)->GetFloatArrayElements(env, {p.name}, 0) : 0;"); post.append(f"  if ({p.name}) (*env)->ReleaseFloatArrayElements(env, {p.name}, {p.name}_p, 0);"); args.append(f"(float*){p.name}_p")
                elif k == "int64ptr":
                    pre.append(f"  jlong* {p.name}_p = {p.name} ? (*env)->GetLongArrayElements(env, {p.name}, 0) : 0;"); post.append(f"  if ({p.name}) (*env)->ReleaseLongArrayElements(env, {p.name}, {p.name}_p, 0);"); args.append(f"(int64_t*){p.name}_p")
                elif k == "handle":
                    args.append(f"({p.ctype})(intptr_t){p.name}")
                elif k == "string":
                    pre.append(f"  const char* {p.name}_p = (*env)->GetStringUTFChars(env, {p.name}, 0);"); post.append(f"  (*env)->ReleaseStringUTFChars(env, {p.name}, {p.name}_p);"); args.append(f"{p.name}_p")
                else:
                    args.append(p.name)
            call, k = f"{f.name}({', '.join(args)})", canonical(f.ret)
            rt = jt[k]
            L.append(f"JNIEXPORT {rt} JNICALL Java_org_torsh_Torsh_{self._lower_camel(f.name)}(JNIEnv* env, jclass cls{ps}) {{")
            L += pre
            if k == "void":
                L.append(f"  {call};"); L += post
            else:
                conv = "(jlong)(intptr_t)" if k == "handle" else ""
                if k == "string":
                    L.append(f"  jstring r = (*env)->NewStringUTF(env, {call});")
                elif k == "floatptr":
                    L.append(f"  jfloatArray r = 0; (void){call}; /* raw data pointers are not exposed to Java: use tensorCopyOut */")
                else:
                    L.append(f"  {rt} r = {conv}{call};")
                L += post + ["  return r;"]
            L += ["}", ""]
        return "\n".join(L)

    @staticmethod
    def _lower_camel(n): c = _camel(n); return c[0].lower() + c[1:]

    def julia(self) -> str:
        L = ["module Torsh", "", f'const lib = "lib{self.lib}"', ""]
        for f in self.fns:
            names = ", ".join(p.name for p in f.params)
            tys = ", ".join(lang_type(p.ctype, "julia") for p in f.params) + ("," if len(f.params) == 1 else "")
            L.append(f"{f.name.removeprefix('torsh_')}({names}) = ccall((:{f.name}, lib), {lang_type(f.ret, 'julia')}, ({tys}){', ' + names if names else ''})")
        L += ["", "mutable struct Tensor", "    handle::Ptr{Cvoid}", "    function Tensor(h::Ptr{Cvoid})", '        h == C_NULL && error(unsafe_string(get_last_error()))', "        t = new(h); finalizer(x -> tensor_free(x.handle), t); t", "    end", "end",
              "Tensor(data::Array{Float32}) = Tensor(tensor_new(pointer(permutedims(data, reverse(1:ndims(data)))), pointer(Int64[size(data)...]), Cint(ndims(data))))", "Base.:+(a::Tensor, b::Tensor) = Tensor(tensor_add(a.handle, b.handle))",
              "Base.:*(a::Tensor, b::Tensor) = Tensor(tensor_matmul(a.handle, b.handle))", "", "end"]
        return "\n".join(L) + "\n"

    def lua(self) -> str:
        decl = "\n".join(f"  {lang_type(f.ret, 'lua')} {f.name}({', '.join(lang_type(p.ctype, 'lua') + ' ' + p.name for p in f.params) or 'void'});" for f in self.fns)
        fns = "\n".join(f"function M.{f.name.removeprefix('torsh_')}(...) return C.{f.name}(...) end" for f in self.fns)
        return (f'local ffi = require("ffi")\nffi.cdef[[\n{decl}\n]]\nlocal C = ffi.load("{self.lib}")\nlocal M = {{}}\n{fns}\n\nlocal Tensor = {{}}\nTensor.__index = Tensor\n'
                "function M.tensor(data, shape)\n  local d = ffi.new(\"float[?]\", #data, data)\n  local s = ffi.new(\"int64_t[?]\", #shape, shape)\n  local h = C.torsh_tensor_new(d, s, #shape)\n  if h == nil then error(ffi.string(C.torsh_get_last_error())) end\n"
                "  return setmetatable({handle = ffi.gc(h, C.torsh_tensor_free)}, Tensor)\nend\nTensor.__add = function(a, b) return setmetatable({handle = ffi.gc(C.torsh_tensor_add(a.handle, b.handle), C.torsh_tensor_free)}, Tensor) end\nreturn M\n")

    def matlab(self) -> str:
        L = ["function [methodinfo, structs, enuminfo, ThunkLibName] = torsh_proto", "% Prototype file for loadlibrary: loadlibrary('lib" + self.lib + "', @torsh_proto)", "structs = []; enuminfo = []; ThunkLibName = '';", "fcns = struct('name', {{}}, 'calltype', {{}}, 'LHS', {{}}, 'RHS', {{}});"]
        for i, f in enumerate(self.fns, 1):
            rhs = ", ".join(f"'{lang_type(p.ctype, 'matlab')}'" for p in f.params)
            L.append(f"fcns.name{{{i}}} = '{f.name}'; fcns.calltype{{{i}}} = 'cdecl'; fcns.LHS{{{i}}} = '{lang_type(f.ret, 'matlab')}'; fcns.RHS{{{i}}} = {{{rhs}}};")
        L += ["methodinfo = fcns;", "end"]
        return "\n".join(L) + "\n"

    def nodejs(self) -> str:
        L = ["'use strict';", "const koffi = require('koffi');", f"const lib = koffi.load(process.env.TORSH_LIBRARY || 'lib{self.lib}.so');", "const api = {};"]
        for f in self.fns:
            L.append(f"api.{self._lower_camel(f.name)} = lib.func('{f.name}', {lang_type(f.ret, 'node')}, [{', '.join(lang_type(p.ctype, 'node') for p in f.params)}]);")
        L += ["", "class Tensor {", "  constructor(handle) { if (!handle) throw new Error(api.getLastError()); this.handle = handle; }", "  static from(data, shape) { return new Tensor(api.tensorNew(Float32Array.from(data), BigInt64Array.from(shape.map(BigInt)), shape.length)); }",
              "  add(o) { return new Tensor(api.tensorAdd(this.handle, o.handle)); }", "  matmul(o) { return new Tensor(api.tensorMatmul(this.handle, o.handle)); }", "  free() { api.tensorFree(this.handle); this.handle = null; }", "}", "module.exports = { api, Tensor };"]
        return "\n".join(L) + "\n"

    def typescript(self) -> str:
        L = ["export interface TorshApi {"] + [f"  {self._lower_camel(f.name)}({', '.join(p.name + ': ' + lang_type(p.ctype, 'ts') for p in f.params)}): {lang_type(f.ret, 'ts')};" for f in self.fns] + ["}", "export declare const api: TorshApi;",
             "export declare class Tensor {", "  static from(data: ArrayLike<number>, shape: number[]): Tensor;", "  add(o: Tensor): Tensor;", "  matmul(o: Tensor): Tensor;", "  free(): void;", "}"]
        return "\n".join(L) + "\n"

    def r(self) -> str:
        L = [f'dyn.load(Sys.getenv("TORSH_LIBRARY", "lib{self.lib}_r.so"))', "# Every wrapper calls a shim of the same name with an R_ prefix (.Call convention: SEXP in, SEXP out)."]
        for f in self.fns:
            names = ", ".join(p.name for p in f.params)
            L.append(f"{f.name} <- function({names}) .Call(\"R_{f.name}\"{', ' + names if names else ''})")
        L += ["", "torsh_tensor <- function(x) {", "  h <- torsh_tensor_new(as.numeric(aperm(x)), as.numeric(dim(x)), length(dim(x)))", '  structure(list(handle = h), class = "torsh_tensor")', "}",
              '"+.torsh_tensor" <- function(a, b) structure(list(handle = torsh_tensor_add(a$handle, b$handle)), class = "torsh_tensor")']
        return "\n".join(L) + "\n"

    def ruby(self) -> str:
        L = ["require 'ffi'", "", "module Torsh", "  extend FFI::Library", f"  ffi_lib ENV.fetch('TORSH_LIBRARY', '{self.lib}')"]
        for f in self.fns:
            L.append(f"  attach_function :{f.name}, [{', '.join(lang_type(p.ctype, 'ruby') for p in f.params)}], {lang_type(f.ret, 'ruby')}")
        L += ["", "  class Tensor", "    attr_reader :handle", "    def initialize(handle)", "      raise Torsh.torsh_get_last_error if handle.null?", "      @handle = FFI::AutoPointer.new(handle, Torsh.method(:torsh_tensor_free))", "    end",
              "    def +(other) = Tensor.new(Torsh.torsh_tensor_add(@handle, other.handle))", "  end", "end"]
        return "\n".join(L) + "\n"

    def swift(self) -> str:
        L = ["// module.modulemap:  module CTorsh { header \"torsh.h\" link \"" + self.lib + "\" export * }", "import CTorsh", "", "public enum TorshError: Error { case failed(String) }", "",
             "@inline(__always) func check(_ status: Int32) throws { if status != 0 { throw TorshError.failed(String(cString: torsh_get_last_error())) } }", "", "public final class Tensor {", "    let handle: OpaquePointer",
             "    init(_ h: OpaquePointer?) throws { guard let h = h else { throw TorshError.failed(String(cString: torsh_get_last_error())) }; handle = h }", "    deinit { torsh_tensor_free(handle) }",
             "    public convenience init(_ data: [Float], shape: [Int64]) throws { try self.init(torsh_tensor_new(data, shape, Int32(shape.count))) }"]
        for f in self.fns:
            if f.name.startswith("torsh_tensor_") and canonical(f.ret) == "handle" and f.params and all(canonical(p.ctype) in ("handle", "int", "float") for p in f.params) and canonical(f.params[0].ctype) == "handle":
                rest = f.params[1:]
                sig = ", ".join(f"{'_ ' if i == 0 else ''}{p.name}: {'Tensor' if canonical(p.ctype) == 'handle' else lang_type(p.ctype, 'swift')}" for i, p in enumerate(rest))
                args = ", ".join(["handle"] + [f"{p.name}.handle" if canonical(p.ctype) == "handle" else p.name for p in rest])
                L.append(f"    public func {self._lower_camel(f.name.replace('torsh_tensor_', 'torsh_'))}({sig}) throws -> Tensor {{ try Tensor({f.name}({args})) }}")
        L += ["}"]
        return "\n".join(L) + "\n"

    def wasm(self) -> str:
        exported = ", ".join(f"'_{f.name}'" for f in self.fns)
        ct = lambda c: {"string": "'string'", "void": "null"}.get(canonical(c), "'number'")
        wraps = "\n".join(f"  api.{self._lower_camel(f.name)} = Module.cwrap('{f.name}', {ct(f.ret)}, [{', '.join(ct(p.ctype) for p in f.params)}]);" for f in self.fns)
        return (f"// emcc ... -sEXPORTED_FUNCTIONS=\"[{exported}, '_malloc', '_free']\" -sEXPORTED_RUNTIME_METHODS=\"['cwrap','HEAPF32','HEAP64']\"\nexport function bind(Module) {{\n  const api = {{}};\n{wraps}\n"
                "  api.tensorFrom = (data, shape) => {\n    const d = Module._malloc(4 * data.length), s = Module._malloc(8 * shape.length);\n    Module.HEAPF32.set(data, d >> 2); Module.HEAP64.set(shape.map(BigInt), s >> 3);\n"
                "    const h = api.tensorNew(d, s, shape.length); Module._free(d); Module._free(s);\n    if (!h) throw new Error(api.getLastError());\n    return h;\n  };\n  return api;\n}\n")


# ================================================================================================ documentation and tests
def generate_api_docs(functions: Sequence[CFunction] | None = None, title: str = "C API reference") -> str:
    fns = list(functions or parse_header())
    groups: dict[str, list] = {}
    for f in fns:
        groups.setdefault(f.group, []).append(f)
    L = [f"# {title}", "", f"{len(fns)} functions. A handle-returning function yields `NULL` on failure and a `TorshStatus` function a non-zero code; the message is read with `torsh_get_last_error()`.", ""]
    L += ["| group | functions |", "|---|---|"] + [f"| [{g}](#{g}) | {len(v)} |" for g, v in groups.items()] + [""]
    for g, v in groups.items():
        L += [f"## {g}", ""]
        for f in v:
            L += [f"### `{f.name}`", "", "```c", f.signature() + ";", "```", ""]
            if f.doc:
                L += [f.doc, ""]
            if f.params:
                L += ["| parameter | type |", "|---|---|"] + [f"| `{p.name}` | `{p.ctype}` |" for p in f.params] + [""]
    return "\n".join(L)


def generate_tests(functions: Sequence[CFunction] | None = None, binding_module: str = "torsh_ffi") -> str:
    """pytest source for the generated ctypes binding: every unary and binary tensor function is called on small inputs and
    checked for a live result of the right size; every reduction for one element; status functions for success."""
    fns = list(functions or parse_header())
    is_t = lambda p: p.ctype.replace("const ", "").strip() == "TorshTensor*"
    unary = [f.name.removeprefix("torsh_") for f in fns if f.ret == "TorshTensor*" and len(f.params) == 1 and is_t(f.params[0]) and not f.name.endswith("_all") and f.name not in ("torsh_tensor_clone", "torsh_tensor_detach")]
    binary = [f.name.removeprefix("torsh_") for f in fns if f.ret == "TorshTensor*" and len(f.params) == 2 and all(is_t(p) for p in f.params) and "matmul" not in f.name]
    reduce_all = [f.name.removeprefix("torsh_") for f in fns if f.ret == "TorshTensor*" and f.name.endswith("_all")]
    getters = [f.name.removeprefix("torsh_") for f in fns if f.ret == "int" and not f.params]
    return f'''"""Generated smoke tests of the C API through the generated binding."""
import ctypes
import os

import pytest

import {binding_module} as binding

api = binding.load(os.environ["TORSH_LIBRARY"])


def make(values, shape):
    data = (ctypes.c_float * len(values))(*values)
    dims = (ctypes.c_int64 * len(shape))(*shape)
    return api.tensor_new(data, dims, len(shape))


@pytest.mark.parametrize("name", {unary!r})
def test_unary(name):
    t = make([0.5, 1.0, 1.5, 2.0, 2.5, 3.0], [2, 3])
    r = getattr(api, name)(t)
    assert api.tensor_numel(r) == 6 and api.tensor_ndim(r) == 2
    api.tensor_free(r); api.tensor_free(t)


@pytest.mark.parametrize("name", {binary!r})
def test_binary(name):
    a, b = make([1.0, 2.0, 3.0, 4.0], [2, 2]), make([4.0, 3.0, 2.0, 1.0], [2, 2])
    r = getattr(api, name)(a, b)
    assert api.tensor_numel(r) == 4
    with pytest.raises(binding.TorshError):
        getattr(api, name)(a, make([1.0, 2.0, 3.0], [3]))
    for t in (a, b, r):
        api.tensor_free(t)


@pytest.mark.parametrize("name", {reduce_all!r})
def test_reduce_all(name):
    t = make([1.0, 2.0, 3.0, 6.0], [4])
    r = getattr(api, name)(t)
    assert api.tensor_numel(r) == 1 and api.tensor_data(r)[0] in (12.0, 3.0, 6.0, 1.0)


@pytest.mark.parametrize("name", {getters!r})
def test_getter(name):
    assert isinstance(getattr(api, name)(), int)


def test_status_and_strings():
    api.init()
    assert api.version().decode().count(".") == 2
    api.set_num_threads(2)
    assert api.get_num_threads() == 2
'''


# ================================================================================================ call batching
class CallBatcher:
    """Queues element-wise calls on handles and executes them in one pass; identical sub-calls are executed once and results
    no later call uses are freed immediately, so a chain costs one round of crossings instead of one per intermediate
    the caller would otherwise hold."""

    def __init__(self, api): self.api, self.queue, self.crossings = api, [], 0
    def call(self, name: str, *args) -> int: self.queue.append((name, args)); return len(self.queue) - 1

    def run(self, keep: Sequence[int]):
        canon, memo, plan = {}, {}, []
        for i, (name, args) in enumerate(self.queue):                               # resolve duplicates first, so that lifetimes are those of the shared result
            cargs = tuple(_Ref(canon[a.index]) if isinstance(a, _Ref) else a for a in args)
            key = (name, tuple(("r", a.index) if isinstance(a, _Ref) else ("v", getattr(a, "value", a)) for a in cargs))
            canon[i] = memo.setdefault(key, i)
            if canon[i] == i:
                plan.append((i, name, cargs))
        kept = {canon[k] for k in keep}
        last_use = {a.index: i for i, _, cargs in plan for a in cargs if isinstance(a, _Ref)}
        results = {}
        for i, name, cargs in plan:
            results[i] = getattr(self.api, name)(*[results[a.index] if isinstance(a, _Ref) else a for a in cargs]); self.crossings += 1
            for idx in {a.index for a in cargs if isinstance(a, _Ref)}:
                if last_use[idx] == i and idx not in kept:
                    self.api.tensor_free(results.pop(idx)); self.crossings += 1
        self.queue = []
        return [results[canon[k]] for k in keep]

    def ref(self, index: int) -> "_Ref": return _Ref(index)


@dataclass(frozen=True)
class _Ref:
    index: int


# ================================================================================================ NumPy protocol
_UFUNCS = {np.add: torch.add, np.subtract: torch.sub, np.multiply: torch.mul, np.true_divide: torch.div, np.exp: torch.exp, np.log: torch.log, np.sqrt: torch.sqrt, np.tanh: torch.tanh, np.maximum: torch.maximum,
           np.minimum: torch.minimum, np.negative: torch.neg, np.abs: torch.abs, np.sin: torch.sin, np.cos: torch.cos, np.power: torch.pow, np.matmul: torch.matmul, np.greater: torch.gt, np.less: torch.lt, np.equal: torch.eq}
_FUNCTIONS: dict = {}


def implements(np_function):
    def deco(fn): _FUNCTIONS[np_function] = fn; return fn
    return deco


class NumpyCompatibleTensor:
    """Tensor wrapper NumPy treats as one of its own: ufuncs and the registered functions run in torch and return the
    wrapper, ``np.asarray`` shares memory on the host."""
    __array_priority__ = 100

    def __init__(self, t): self.t = t if isinstance(t, torch.Tensor) else torch.as_tensor(np.asarray(t))
    def __array__(self, dtype=None, copy=None): a = self.t.detach().cpu().numpy(); return a.astype(dtype) if dtype is not None else a
    @property
    def shape(self): return tuple(self.t.shape)
    @property
    def dtype(self): return np.dtype(str(self.t.dtype).replace("torch.", ""))
    @property
    def ndim(self): return self.t.dim()
    @property
    def T(self): return NumpyCompatibleTensor(self.t.T)
    def __len__(self): return len(self.t)
    def __getitem__(self, i): return NumpyCompatibleTensor(self.t[i])
    def __repr__(self): return f"NumpyCompatibleTensor({self.t!r})"
    @staticmethod
    def _un(x): return x.t if isinstance(x, NumpyCompatibleTensor) else torch.as_tensor(x) if isinstance(x, np.ndarray) else x

    def __array_ufunc__(self, ufunc, method, *inputs, **kw):
        if method == "reduce" and ufunc in (np.add, np.maximum, np.minimum, np.multiply):
            f = {np.add: torch.sum, np.maximum: torch.amax, np.minimum: torch.amin, np.multiply: torch.prod}[ufunc]
            ax = kw.get("axis", 0)
            return NumpyCompatibleTensor(f(self._un(inputs[0])) if ax is None else f(self._un(inputs[0]), dim=ax, keepdim=kw.get("keepdims", False)))
        if method != "__call__" or ufunc not in _UFUNCS:
            return NotImplemented
        return NumpyCompatibleTensor(_UFUNCS[ufunc](*[self._un(i) for i in inputs]))

    def __array_function__(self, func, types, args, kwargs):
        if func not in _FUNCTIONS:
            return NotImplemented
        return _FUNCTIONS[func](*args, **kwargs)

    for _n, _f in (("__add__", torch.add), ("__sub__", torch.sub), ("__mul__", torch.mul), ("__truediv__", torch.div), ("__matmul__", torch.matmul)):
        locals()[_n] = (lambda f: lambda self, o: NumpyCompatibleTensor(f(self.t, NumpyCompatibleTensor._un(o))))(_f)
    del _n, _f


_W, _U = NumpyCompatibleTensor, NumpyCompatibleTensor._un
implements(np.sum)(lambda a, axis=None, keepdims=False, **k: _W(_U(a).sum() if axis is None else _U(a).sum(dim=axis, keepdim=keepdims)))
implements(np.mean)(lambda a, axis=None, keepdims=False, **k: _W(_U(a).mean() if axis is None else _U(a).mean(dim=axis, keepdim=keepdims)))
implements(np.concatenate)(lambda arrs, axis=0, **k: _W(torch.cat([_U(a) for a in arrs], dim=axis)))
implements(np.stack)(lambda arrs, axis=0, **k: _W(torch.stack([_U(a) for a in arrs], dim=axis)))
implements(np.reshape)(lambda a, shape=None, *r, **k: _W(_U(a).reshape(shape if shape is not None else k["newshape"])))
implements(np.transpose)(lambda a, axes=None: _W(_U(a).permute(*axes) if axes is not None else _U(a).permute(*reversed(range(_U(a).dim())))))
implements(np.dot)(lambda a, b, **k: _W(torch.matmul(_U(a), _U(b))))
implements(np.where)(lambda c, a, b: _W(torch.where(_U(c).bool(), torch.as_tensor(_U(a)), torch.as_tensor(_U(b)))))
implements(np.argmax)(lambda a, axis=None, **k: _W(_U(a).argmax() if axis is None else _U(a).argmax(dim=axis)))
implements(np.clip)(lambda a, a_min=None, a_max=None, **k: _W(_U(a).clamp(a_min, a_max)))
implements(np.linalg.norm)(lambda a, ord=None, axis=None, keepdims=False: _W(torch.linalg.norm(_U(a), ord=ord, dim=axis, keepdim=keepdims)))
implements(np.allclose)(lambda a, b, rtol=1e-5, atol=1e-8, **k: bool(torch.allclose(torch.as_tensor(_U(a)), torch.as_tensor(_U(b)), rtol=rtol, atol=atol)))

NUMPY_DTYPES = {np.dtype("float32"): torch.float32, np.dtype("float64"): torch.float64, np.dtype("float16"): torch.float16, np.dtype("int8"): torch.int8, np.dtype("int16"): torch.int16, np.dtype("int32"): torch.int32,
                np.dtype("int64"): torch.int64, np.dtype("uint8"): torch.uint8, np.dtype("bool"): torch.bool, np.dtype("complex64"): torch.complex64, np.dtype("complex128"): torch.complex128}


def from_numpy(a: np.ndarray, copy: bool = False) -> torch.Tensor:
    """Zero-copy when the array is writable with non-negative strides; otherwise (or when ``copy``) a contiguous copy."""
    if a.dtype not in NUMPY_DTYPES:
        raise TypeError(f"no tensor dtype for {a.dtype}")
    ok = a.flags.writeable and all(s >= 0 for s in a.strides) and a.dtype.isnative
    return torch.from_numpy(a) if ok and not copy else torch.from_numpy(np.ascontiguousarray(a).copy())


# ================================================================================================ pandas
def dataframe_to_tensors(df, target: str | None = None, categorical: str = "codes", dtype=torch.float32) -> dict:
    """Numeric columns stacked into ``features``; categoricals / strings become integer codes (or one-hot blocks); booleans 0/1;
    datetimes seconds since the epoch; missing numeric values become NaN.  ``columns`` and ``categories`` allow the way back."""
    import pandas as pd
    cols, names, cats = [], [], {}
    for c in df.columns:
        if c == target:
            continue
        s = df[c]
        if isinstance(s.dtype, pd.CategoricalDtype) or s.dtype == object or pd.api.types.is_string_dtype(s.dtype):
            cat = s.astype("category")
            cats[c] = list(cat.cat.categories)
            codes = torch.as_tensor(cat.cat.codes.to_numpy().astype(np.int64))
            if categorical == "onehot":
                oh = torch.nn.functional.one_hot(codes.clamp(min=0), len(cats[c])).to(dtype) * (codes >= 0)[:, None]
                cols += list(oh.T); names += [f"{c}={k}" for k in cats[c]]
            else:
                cols.append(codes.to(dtype)); names.append(c)
        elif pd.api.types.is_datetime64_any_dtype(s.dtype):
            cols.append(torch.as_tensor((s.astype("datetime64[ns]").astype("int64") // 10 ** 9).to_numpy().copy()).to(dtype)); names.append(c)
        else:
            cols.append(torch.as_tensor(s.to_numpy(dtype=np.float64, na_value=np.nan).copy()).to(dtype)); names.append(c)
    out = {"features": torch.stack(cols, 1) if cols else torch.empty(len(df), 0, dtype=dtype), "columns": names, "categories": cats, "index": df.index.to_numpy()}
    if target is not None:
        t = df[target]
        if t.dtype == object or isinstance(t.dtype, pd.CategoricalDtype) or pd.api.types.is_string_dtype(t.dtype):
            cat = t.astype("category"); out["target"], out["target_classes"] = torch.as_tensor(cat.cat.codes.to_numpy().astype(np.int64)), list(cat.cat.categories)
        else:
            out["target"] = torch.as_tensor(t.to_numpy())
    return out


def tensor_to_dataframe(t: torch.Tensor, columns: Sequence[str] | None = None, categories: dict | None = None, index=None):
    import pandas as pd
    a = t.detach().cpu().numpy()
    df = pd.DataFrame(a if a.ndim == 2 else a.reshape(len(a), -1), columns=list(columns) if columns else None, index=index)
    for c, names in (categories or {}).items():
        if c in df:
            df[c] = pd.Categorical.from_codes(df[c].astype(int), names)
    return df


class DataFrameDataset(torch.utils.data.Dataset):
    def __init__(self, df, target: str, **kw): self.d = dataframe_to_tensors(df, target, **kw)
    def __len__(self): return len(self.d["features"])
    def __getitem__(self, i): return self.d["features"][i], self.d["target"][i]


# ================================================================================================ SciPy
def scipy_minimize(fn: Callable[[torch.Tensor], torch.Tensor], x0: torch.Tensor, method: str = "L-BFGS-B", **kw):
    """``scipy.optimize.minimize`` with the objective written on tensors and its gradient supplied by autograd."""
    from scipy.optimize import minimize
    def fg(v):
        x = torch.tensor(v, dtype=torch.float64).reshape(x0.shape).requires_grad_(True)
        y = fn(x); g, = torch.autograd.grad(y, x)
        return float(y.detach()), g.reshape(-1).numpy()
    r = minimize(fg, x0.detach().double().reshape(-1).numpy(), jac=True, method=method, **kw)
    r.x_tensor = torch.as_tensor(r.x).reshape(x0.shape).to(x0.dtype)
    return r


def scipy_solve_ivp(f: Callable[[float, torch.Tensor], torch.Tensor], t_span, y0: torch.Tensor, **kw):
    from scipy.integrate import solve_ivp
    r = solve_ivp(lambda t, y: f(t, torch.as_tensor(y)).numpy(), t_span, y0.double().numpy(), **kw)
    return torch.as_tensor(r.t), torch.as_tensor(r.y).T


def to_scipy_sparse(t: torch.Tensor):
    from scipy import sparse
    c = t.to_sparse_coo().coalesce() if not t.is_sparse else t.coalesce()
    i = c.indices().numpy()
    return sparse.coo_matrix((c.values().numpy(), (i[0], i[1])), shape=tuple(c.shape)).tocsr()


def from_scipy_sparse(m) -> torch.Tensor:
    c = m.tocoo()
    return torch.sparse_coo_tensor(torch.as_tensor(np.stack([c.row, c.col]).astype(np.int64)), torch.as_tensor(c.data), c.shape).coalesce()


def scipy_function(name: str) -> Callable:
    """``scipy.special`` / ``scipy.signal`` / ``scipy.linalg`` function lifted to tensors (host round trip, no gradient)."""
    import importlib
    mod, fn = name.rsplit(".", 1)
    f = getattr(importlib.import_module(f"scipy.{mod}"), fn)
    conv = lambda r: torch.as_tensor(np.asarray(r)) if isinstance(r, (np.ndarray, np.generic)) else tuple(conv(x) for x in r) if isinstance(r, tuple) else r
    return lambda *a, **k: conv(f(*[x.detach().cpu().numpy() if isinstance(x, torch.Tensor) else x for x in a], **k))


# ================================================================================================ plots and notebook views
_RAMP = " .:-=+*#%@"


def ascii_heatmap(t: torch.Tensor, width: int = 40, height: int = 16) -> str:
    a = torch.nn.functional.adaptive_avg_pool2d(t.detach().float()[None, None], (min(height, t.shape[0]), min(width, t.shape[1])))[0, 0]
    lo, hi = float(a.min()), float(a.max())
    idx = ((a - lo) / (hi - lo if hi > lo else 1.0) * (len(_RAMP) - 1)).round().long()
    return "\n".join("".join(_RAMP[i] for i in row) for row in idx.tolist())


def ascii_histogram(t: torch.Tensor, bins: int = 10, width: int = 40) -> str:
    v = t.detach().float().flatten()
    lo, hi = float(v.min()), float(v.max())
    h = torch.histc(v, bins, lo, hi)
    step = (hi - lo) / bins
    return "\n".join(f"{lo + i * step:>10.3g} | {'#' * int(round(float(c) / float(h.max()) * width))} {int(c)}" for i, c in enumerate(h))


def heatmap_svg(t: torch.Tensor, cell: int = 12, title: str = "") -> str:
    a = t.detach().float()
    lo, hi = float(a.min()), float(a.max())
    n = ((a - lo) / (hi - lo if hi > lo else 1.0)).tolist()
    def colour(v):                                                                   # blue -> white -> red
        r, b = (255, int(255 * (1 - (v - 0.5) * 2))) if v >= 0.5 else (int(255 * v * 2), 255)
        return f"#{r:02x}{min(r, b):02x}{b:02x}"
    rects = "".join(f'<rect x="{j * cell}" y="{i * cell + 16}" width="{cell}" height="{cell}" fill="{colour(v)}"><title>[{i},{j}] {float(a[i, j]):.4g}</title></rect>' for i, row in enumerate(n) for j, v in enumerate(row))
    return f'<svg xmlns="http://www.w3.org/2000/svg" width="{a.shape[1] * cell}" height="{a.shape[0] * cell + 16}"><text x="0" y="12" font-size="11">{html.escape(title)}</text>{rects}</svg>'


def training_curves_svg(history: dict[str, Sequence[float]], title: str = "training") -> str:
    from .utils.bench_suite import Chart
    ch = Chart(title, x_label="step", y_label="value")
    for k, v in history.items():
        ch.add_series(k, range(len(v)), v)
    return ch.to_svg()


class TensorView:
    """Notebook representation: shape / dtype / statistics table and, for matrices of moderate size, a heat map."""

    def __init__(self, t: torch.Tensor, name: str = "tensor", max_cells: int = 4096): self.t, self.name, self.max_cells = t, name, max_cells

    def _repr_html_(self) -> str:
        t = self.t.detach()
        rows = [("shape", list(t.shape)), ("dtype", str(t.dtype).replace("torch.", "")), ("device", t.device), ("bytes", f"{t.numel() * t.element_size():,}")]
        if t.numel() and (t.is_floating_point() or not t.is_complex()):
            f = t.double()
            rows += [("min", f"{float(f.min()):.4g}"), ("max", f"{float(f.max()):.4g}"), ("mean", f"{float(f.mean()):.4g}"), ("std", f"{float(f.std()):.4g}" if t.numel() > 1 else "0"), ("nan", int(torch.isnan(f).sum()))]
        table = "<table>" + "".join(f"<tr><th>{k}</th><td>{html.escape(str(v))}</td></tr>" for k, v in rows) + "</table>"
        plot = heatmap_svg(t.float(), title=self.name) if t.dim() == 2 and 0 < t.numel() <= self.max_cells else f"<pre>{html.escape(ascii_histogram(t))}</pre>" if t.numel() > 1 and not t.is_complex() else ""
        return f"<div class='torsh-tensor'><b>{html.escape(self.name)}</b>{table}{plot}</div>"

    def _repr_mimebundle_(self, include=None, exclude=None): return {"text/html": self._repr_html_(), "text/plain": repr(self.t)}


class ProgressView:
    def __init__(self, total: int, label: str = ""): self.total, self.n, self.label = total, 0, label
    def update(self, k: int = 1): self.n = min(self.total, self.n + k); return self
    def _repr_html_(self): return f"<label>{html.escape(self.label)} <progress value='{self.n}' max='{self.total}'></progress> {self.n}/{self.total}</label>"
    def __str__(self): w = 30; f = int(w * self.n / max(self.total, 1)); return f"{self.label} [{'=' * f}{' ' * (w - f)}] {self.n}/{self.total}"


# ================================================================================================ migration from other frameworks
_MODULE_MAP = {"pytorch": {"torch.nn.functional": "torsh_b200.nn.functional", "torch.nn": "torsh_b200.nn", "torch.optim": "torsh_b200.optim", "torch.utils.data": "torsh_b200.data", "torch.distributed": "torsh_b200.parallel",
                           "torch.autograd": "torsh_b200.autograd", "torch.fx": "torsh_b200.fx", "torch.jit": "torsh_b200.jit", "torch.linalg": "torsh_b200.linalg", "torch.sparse": "torsh_b200.sparse", "torchvision": "torsh_b200.vision",
                           "torchtext": "torsh_b200.text", "torch": "rstorch"},
               "numpy": {"numpy.linalg": "torsh_b200.linalg", "numpy.fft": "torsh_b200.signal", "numpy": "rstorch"},
               "tensorflow": {"tensorflow.keras.layers": "torsh_b200.nn", "tensorflow.keras.optimizers": "torsh_b200.optim", "tensorflow.data": "torsh_b200.data", "tensorflow": "rstorch"}}
_ATTR_MAP = {"numpy": {"array": "tensor", "concatenate": "cat", "expand_dims": "unsqueeze", "ndarray": "Tensor", "float32": "float32", "dot": "matmul", "power": "pow", "absolute": "abs"},
             "tensorflow": {"constant": "tensor", "concat": "cat", "reduce_sum": "sum", "reduce_mean": "mean", "reduce_max": "amax", "expand_dims": "unsqueeze", "Dense": "Linear", "Adam": "Adam", "SGD": "SGD", "math": None},
             "pytorch": {}}
_KWARG_MAP = {"numpy": {"axis": "dim", "keepdims": "keepdim"}, "tensorflow": {"axis": "dim", "keepdims": "keepdim", "learning_rate": "lr", "units": "out_features"}, "pytorch": {}}


class _Migrator(ast.NodeTransformer):
    def __init__(self, framework): self.fw, self.mods, self.attrs, self.kw, self.aliases, self.changes, self.manual = framework, _MODULE_MAP[framework], _ATTR_MAP[framework], _KWARG_MAP[framework], {}, [], []

    def _map_module(self, name):
        for src in sorted(self.mods, key=len, reverse=True):
            if name == src or name.startswith(src + "."):
                return self.mods[src] + name[len(src):]
        return None

    def visit_Import(self, node):
        for a in node.names:
            new = self._map_module(a.name)
            if new:
                self.changes.append((node.lineno, f"import {a.name} -> import {new}"))
                self.aliases[a.asname or a.name.split(".")[0]] = True
                if a.asname is None and "." not in a.name:
                    a.asname = a.name
                a.name = new
        return node

    def visit_ImportFrom(self, node):
        new = self._map_module(node.module or "")
        if new:
            self.changes.append((node.lineno, f"from {node.module} -> from {new}")); node.module = new
            for a in node.names:
                if self.attrs.get(a.name):
                    a.asname, a.name = a.asname or a.name, self.attrs[a.name]
        return node

    def visit_Call(self, node):
        self.generic_visit(node)
        root = node.func
        while isinstance(root, ast.Attribute):
            root = root.value
        if isinstance(root, ast.Name) and root.id in self.aliases:
            for k in node.keywords:
                if k.arg in self.kw:
                    self.changes.append((node.lineno, f"keyword {k.arg} -> {self.kw[k.arg]}")); k.arg = self.kw[k.arg]
        return node

    def visit_Attribute(self, node):
        self.generic_visit(node)
        root = node.value
        while isinstance(root, ast.Attribute):
            root = root.value
        if isinstance(root, ast.Name) and root.id in self.aliases and node.attr in self.attrs:
            new = self.attrs[node.attr]
            if new is None:
                return node.value                                                  # tf.math.exp -> tf.exp: drop the namespace
            if new != node.attr:
                self.changes.append((node.lineno, f".{node.attr} -> .{new}")); node.attr = new
        if isinstance(root, ast.Name) and root.id in self.aliases and node.attr in ("Session", "placeholder", "GradientTape", "einsum_path", "ctypeslib"):
            self.manual.append((node.lineno, f"{node.attr} has no direct counterpart: rewrite by hand"))
        return node


def migrate_source(code: str, framework: str = "pytorch") -> dict:
    """Rewrites imports, renamed functions and keyword arguments of a program written for another framework; constructs
    without a counterpart are listed for manual work.  Returns the new source and the report."""
    tree = ast.parse(code)
    m = _Migrator(framework)
    tree = ast.fix_missing_locations(m.visit(tree))
    return {"source": ast.unparse(tree) + "\n", "changes": m.changes, "manual": m.manual, "framework": framework}

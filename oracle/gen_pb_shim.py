"""TEST INFRASTRUCTURE ONLY.  Stand-ins for the protoc-generated headers the reference's executor
needs (cudarpc.pb.h, signal.pb.h), made from the reference's own .proto files at build time.

protoc is not available in this environment, and the reference's include/server/cuda_server.hpp
cannot be compiled without the message classes.  This script reads proto/cudarpc.proto and
proto/signal.proto where they lie and writes, for every message, a plain C++ class with the
accessors protoc would generate for the constructs those files use (proto3 scalars, enums,
bytes/string, repeated scalars, repeated bytes, repeated messages) and with real proto3 wire
encoding, so that serialised requests made elsewhere (python protobuf, the library's own codec)
parse here and the responses serialised here parse elsewhere.  Output goes to oracle/_ref/gen/
(git-ignored, like everything built from the reference tree); nothing of the reference is copied
into the repository.

    python oracle/gen_pb_shim.py <reference root> <output directory>
"""
import os
import re
import sys

SCALARS = {
    "int32": ("int32_t", "varint"), "int64": ("int64_t", "varint"), "uint32": ("uint32_t", "varint"),
    "uint64": ("uint64_t", "varint"), "bool": ("bool", "varint"), "float": ("float", "fixed32"),
    "double": ("double", "fixed64"),
}

RUNTIME = r'''
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#ifndef TORPOR_PB_SHIM_RUNTIME_
#define TORPOR_PB_SHIM_RUNTIME_
namespace pbshim {
inline void put_varint(std::string* out, uint64_t v) {
    while (v >= 0x80) { out->push_back((char)(v | 0x80)); v >>= 7; }
    out->push_back((char)v);
}
inline void put_tag(std::string* out, int field, int wire) { put_varint(out, ((uint64_t)field << 3) | (uint64_t)wire); }
inline void put_fixed32(std::string* out, uint32_t v) { out->append((const char*)&v, 4); }
inline void put_fixed64(std::string* out, uint64_t v) { out->append((const char*)&v, 8); }
inline void put_bytes(std::string* out, const std::string& s) { put_varint(out, s.size()); out->append(s); }
struct Reader {
    const unsigned char* p;
    const unsigned char* end;
    bool ok = true;
    Reader(const char* data, size_t n) : p((const unsigned char*)data), end((const unsigned char*)data + n) {}
    bool more() const { return ok && p < end; }
    uint64_t varint() {
        uint64_t v = 0;
        for (int shift = 0; shift < 70; shift += 7) {
            if (p >= end) { ok = false; return 0; }
            unsigned char b = *p++;
            v |= (uint64_t)(b & 0x7f) << shift;
            if (!(b & 0x80)) return v;
        }
        ok = false;
        return 0;
    }
    uint32_t fixed32() { uint32_t v = 0; if (end - p < 4) { ok = false; return 0; } memcpy(&v, p, 4); p += 4; return v; }
    uint64_t fixed64() { uint64_t v = 0; if (end - p < 8) { ok = false; return 0; } memcpy(&v, p, 8); p += 8; return v; }
    std::string bytes() {
        uint64_t n = varint();
        if (!ok || (uint64_t)(end - p) < n) { ok = false; return std::string(); }
        std::string s((const char*)p, (size_t)n);
        p += n;
        return s;
    }
    void skip(int wire) {
        if (wire == 0) varint();
        else if (wire == 1) fixed64();
        else if (wire == 2) bytes();
        else if (wire == 5) fixed32();
        else ok = false;
    }
};
}  // namespace pbshim
#endif
'''


def parse_proto(path):
    text = re.sub(r"//[^\n]*", "", open(path).read())
    package = re.search(r"package\s+([A-Za-z0-9_.]+)\s*;", text).group(1)
    enums, messages = [], []
    for m in re.finditer(r"enum\s+(\w+)\s*\{([^}]*)\}", text):
        values = re.findall(r"(\w+)\s*=\s*(-?\d+)\s*;", m.group(2))
        enums.append((m.group(1), values))
    for m in re.finditer(r"message\s+(\w+)\s*\{([^}]*)\}", text):
        fields = []
        for f in re.finditer(r"(repeated\s+)?([A-Za-z0-9_.]+)\s+(\w+)\s*=\s*(\d+)\s*;", m.group(2)):
            # protoc names the C++ accessors after the lower-cased field name
            fields.append((bool(f.group(1)), f.group(2), f.group(3).lower(), int(f.group(4))))
        messages.append((m.group(1), sorted(fields, key=lambda x: x[3])))
    return package, enums, messages


def emit(package, enums, messages):
    enum_names = {e[0] for e in enums}
    msg_names = {m[0] for m in messages}
    out = [RUNTIME, f"namespace {package} {{"]
    for name, values in enums:
        out.append(f"enum {name} : int {{")
        out += [f"    {n} = {v}," for n, v in values]
        out.append("};")
    for name, _ in messages:
        out.append(f"class {name};")
    for name, fields in messages:
        body, parse, ser, clear = [], [], [], []
        for rep, typ, fname, num in fields:
            member = f"{fname}_"
            if typ in SCALARS or typ in enum_names:
                ctype, wire = SCALARS.get(typ, (typ, "varint"))
                wire_no = {"varint": 0, "fixed64": 1, "fixed32": 5}[wire]
                if wire == "varint":
                    put = lambda v: f"pbshim::put_varint(out, (uint64_t)(int64_t)({v}))" if typ in ("int32", "int64") or typ in enum_names \
                        else f"pbshim::put_varint(out, (uint64_t)({v}))"
                    get = f"({ctype})r.varint()"
                elif wire == "fixed32":
                    put = lambda v: f"{{ uint32_t w; float f = {v}; memcpy(&w, &f, 4); pbshim::put_fixed32(out, w); }}"
                    get = "[&]{ uint32_t w = r.fixed32(); float f; memcpy(&f, &w, 4); return f; }()"
                else:
                    put = lambda v: f"{{ uint64_t w; double f = {v}; memcpy(&w, &f, 8); pbshim::put_fixed64(out, w); }}"
                    get = "[&]{ uint64_t w = r.fixed64(); double f; memcpy(&f, &w, 8); return f; }()"
                if rep:
                    body += [f"    int {fname}_size() const {{ return (int){member}.size(); }}",
                             f"    {ctype} {fname}(int i) const {{ return {member}[i]; }}",
                             f"    void add_{fname}({ctype} v) {{ {member}.push_back(v); }}",
                             f"    const std::vector<{ctype}>& {fname}() const {{ return {member}; }}",
                             f"    std::vector<{ctype}> {member};"]
                    parse.append(f"            case {num}: if (wire == 2) {{ std::string pk = r.bytes(); pbshim::Reader q(pk.data(), pk.size()); "
                                 f"auto& r0 = r; (void)r0; while (q.more()) {{ auto& r = q; {member}.push_back({get}); }} }} "
                                 f"else {member}.push_back({get}); break;")
                    ser.append(f"        if (!{member}.empty()) {{ std::string pk; {{ std::string* out = &pk; for (auto v : {member}) {put('v')}; }} "
                               f"pbshim::put_tag(out, {num}, 2); pbshim::put_bytes(out, pk); }}")
                    clear.append(f"{member}.clear();")
                else:
                    body += [f"    {ctype} {fname}() const {{ return {member}; }}",
                             f"    void set_{fname}({ctype} v) {{ {member} = v; }}",
                             f"    {ctype} {member} = {ctype}();"]
                    parse.append(f"            case {num}: {member} = {get}; break;")
                    ser.append(f"        if ({member} != {ctype}()) {{ pbshim::put_tag(out, {num}, {wire_no}); {put(member)}; }}")
                    clear.append(f"{member} = {ctype}();")
            elif typ in ("bytes", "string"):
                if rep:
                    body += [f"    int {fname}_size() const {{ return (int){member}.size(); }}",
                             f"    const std::string& {fname}(int i) const {{ return {member}[i]; }}",
                             f"    void add_{fname}(const std::string& v) {{ {member}.push_back(v); }}",
                             f"    void add_{fname}(const void* p, size_t n) {{ {member}.emplace_back((const char*)p, n); }}",
                             f"    std::string* add_{fname}() {{ {member}.emplace_back(); return &{member}.back(); }}",
                             f"    const std::vector<std::string>& {fname}() const {{ return {member}; }}",
                             f"    std::vector<std::string> {member};"]
                    parse.append(f"            case {num}: {member}.push_back(r.bytes()); break;")
                    ser.append(f"        for (auto& v : {member}) {{ pbshim::put_tag(out, {num}, 2); pbshim::put_bytes(out, v); }}")
                    clear.append(f"{member}.clear();")
                else:
                    body += [f"    const std::string& {fname}() const {{ return {member}; }}",
                             f"    void set_{fname}(const std::string& v) {{ {member} = v; }}",
                             f"    void set_{fname}(const char* v) {{ {member} = v; }}",
                             f"    void set_{fname}(const void* p, size_t n) {{ {member}.assign((const char*)p, n); }}",
                             f"    std::string* mutable_{fname}() {{ return &{member}; }}",
                             f"    std::string {member};"]
                    parse.append(f"            case {num}: {member} = r.bytes(); break;")
                    ser.append(f"        if (!{member}.empty()) {{ pbshim::put_tag(out, {num}, 2); pbshim::put_bytes(out, {member}); }}")
                    clear.append(f"{member}.clear();")
            elif typ in msg_names:
                if not rep:
                    raise SystemExit(f"{name}.{fname}: singular sub-messages are not used by these files; add them here")
                body += [f"    int {fname}_size() const {{ return (int){member}.size(); }}",
                         f"    const {typ}& {fname}(int i) const {{ return {member}[i]; }}",
                         f"    {typ}* add_{fname}();",
                         f"    const std::vector<{typ}>& {fname}() const {{ return {member}; }}",
                         f"    std::vector<{typ}> {member};"]
                parse.append(f"            case {num}: {{ std::string s = r.bytes(); {member}.emplace_back(); {member}.back().ParseFromString(s); }} break;")
                ser.append(f"        for (auto& v : {member}) {{ std::string s; v.SerializeToString(&s); pbshim::put_tag(out, {num}, 2); pbshim::put_bytes(out, s); }}")
                clear.append(f"{member}.clear();")
            else:
                raise SystemExit(f"{name}.{fname}: unknown type {typ}")
        out.append(f"class {name} {{\npublic:")
        out += body
        out.append("    void Clear() { " + " ".join(clear) + " }")
        out.append("    bool ParseFromArray(const void* data, int n) {\n        Clear();\n        pbshim::Reader r((const char*)data, (size_t)n);\n"
                   "        while (r.more()) {\n            uint64_t key = r.varint();\n            if (!r.ok) break;\n"
                   "            int wire = (int)(key & 7);\n            (void)wire;\n            switch ((int)(key >> 3)) {")
        out += parse
        out.append("            default: r.skip(wire); break;\n            }\n        }\n        return r.ok;\n    }")
        out.append("    bool ParseFromString(const std::string& s) { return ParseFromArray(s.data(), (int)s.size()); }")
        out.append("    bool SerializeToString(std::string* out) const {\n        out->clear();\n        AppendTo(out);\n        return true;\n    }")
        out.append("    void AppendTo(std::string* out) const {")
        out += ser
        out.append("    }")
        out.append("    std::string SerializeAsString() const { std::string s; SerializeToString(&s); return s; }")
        out.append("    size_t ByteSizeLong() const { return SerializeAsString().size(); }")
        out.append("};")
    # out-of-line members that need complete types
    for name, fields in messages:
        for rep, typ, fname, num in fields:
            if typ in msg_names and rep:
                out.append(f"inline {typ}* {name}::add_{fname}() {{ {fname}_.emplace_back(); return &{fname}_.back(); }}")
    out.append(f"}}  // namespace {package}")
    return "\n".join(out) + "\n"


def order_messages(messages):
    """Definition order: a message after the messages it holds."""
    names = {m[0] for m in messages}
    done, out = set(), []
    pending = list(messages)
    while pending:
        progressed = False
        for m in list(pending):
            deps = {f[1] for f in m[1] if f[1] in names and f[1] != m[0]}
            if deps <= done:
                out.append(m); done.add(m[0]); pending.remove(m); progressed = True
        if not progressed:
            raise SystemExit("cyclic message definitions")
    return out


def main():
    ref, out_dir = sys.argv[1], sys.argv[2]
    os.makedirs(out_dir, exist_ok=True)
    for stem in ("cudarpc", "signal"):
        package, enums, messages = parse_proto(os.path.join(ref, "proto", stem + ".proto"))
        guard = f"TORPOR_PB_SHIM_{stem.upper()}_H_"
        text = (f"// Generated by oracle/gen_pb_shim.py from proto/{stem}.proto of the reference tree.  Test infrastructure only.\n"
                f"#ifndef {guard}\n#define {guard}\n" + emit(package, enums, order_messages(messages)) + "#endif\n")
        with open(os.path.join(out_dir, stem + ".pb.h"), "w") as f:
            f.write(text)
        # what the reference's cuda_common.hpp does with using-declarations, for every type (the
        # enumerators must stay inside their namespace: several are named like CUDA functions)
        with open(os.path.join(out_dir, stem + ".using.h"), "w") as f:
            f.write("".join(f"using {package}::{n};\n" for n in [e[0] for e in enums] + [m[0] for m in messages]))
        print(f"{stem}.pb.h: {len(enums)} enums, {len(messages)} messages")


if __name__ == "__main__":
    main()

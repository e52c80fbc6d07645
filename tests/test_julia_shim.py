"""The Julia host side (julia/MixtureOfExpertsB200.jl) cannot be executed where this library is
developed, so its binding is checked statically against include/moe_b200.h: every ccall names a
declared entry point and passes the declared number and kind of arguments, and the two structs it
mirrors have the header's fields in the header's order."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "moe_b200.h")
SHIM = os.path.join(ROOT, "julia", "MixtureOfExpertsB200.jl")


def _strip_c_comments(text):
    return re.sub(r"/\*.*?\*/", " ", text, flags=re.S)


def _c_kind(param):
    """'ptr', 'i32', 'i64', 'f32' of one C parameter or return type."""
    p = param.strip()
    if "*" in p:
        return "ptr"
    base = re.sub(r"\bconst\b", "", p).split()
    t = base[0]
    return {"int": "i32", "int32_t": "i32", "int64_t": "i64", "float": "f32", "void": "void"}[t]


def _julia_kind(t):
    t = t.strip()
    if t.startswith(("Ptr{", "Ref{")) or t == "Cstring":
        return "ptr"
    return {"Cint": "i32", "Int32": "i32", "Int64": "i64", "Cfloat": "f32", "Float32": "f32"}[t]


def header_declarations():
    text = _strip_c_comments(open(HEADER).read())
    decls = {}
    for ret, name, params in re.findall(r"^\s*((?:const\s+)?[a-z0-9_]+\s*\*?)\s*(moe_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;", text,
                                        flags=re.M | re.S):
        plist = [q for q in (s.strip() for s in params.replace("\n", " ").split(",")) if q and q != "void"]
        decls[name] = (_c_kind(ret), [_c_kind(q) for q in plist])
    return decls


def shim_ccalls():
    text = open(SHIM).read()
    calls = []
    for m in re.finditer(r"ccall\(\(:(moe_[a-z0-9_]+),\s*LIB\),\s*(\w+),\s*\(([^)]*)\)", text, flags=re.S):
        args = [a for a in (s.strip() for s in m.group(3).replace("\n", " ").split(",")) if a]
        calls.append((m.group(1), _julia_kind(m.group(2)), [_julia_kind(a) for a in args], text[:m.start()].count("\n") + 1))
    return calls


def test_every_ccall_matches_its_declaration():
    decls = header_declarations()
    calls = shim_ccalls()
    assert len(calls) >= 15, "the shim's ccalls were not found: has its calling convention changed?"
    for name, ret, args, line in calls:
        assert name in decls, f"{SHIM}:{line}: {name} is not declared in the header"
        c_ret, c_args = decls[name]
        assert ret == c_ret, f"{SHIM}:{line}: {name} returns {c_ret} in the header, {ret} in the shim"
        assert args == c_args, f"{SHIM}:{line}: {name} takes {c_args} in the header, {args} in the shim"


def _c_struct_fields(name):
    text = _strip_c_comments(open(HEADER).read())
    body = re.search(r"typedef struct \w+\s*\{([^{}]*)\}\s*" + name + r"\s*;", text, flags=re.S).group(1)
    fields = []
    for decl in body.split(";"):
        decl = decl.strip()
        if not decl:
            continue
        m = re.match(r"(.*?)(\w+)$", decl, flags=re.S)
        fields.append((m.group(2), _c_kind(m.group(1))))
    return fields


def _julia_struct_fields(name):
    text = open(SHIM).read()
    body = re.search(r"struct " + name + r"\b[^\n]*\n(.*?)\nend", text, flags=re.S).group(1)
    fields = []
    for decl in re.split(r"[;\n]", body):
        decl = decl.split("#")[0].strip()
        if decl:
            fname, ftype = decl.split("::")
            fields.append((fname.strip(), _julia_kind(ftype)))
    return fields


def test_mirrored_structs_have_the_header_layout():
    assert _julia_struct_fields("CMoeConfig") == _c_struct_fields("moe_config_t")
    assert _julia_struct_fields("CForwardOutputs") == _c_struct_fields("moe_forward_outputs_t")


def test_enum_values_in_the_shim_equal_the_header():
    header = open(HEADER).read()
    shim = open(SHIM).read()
    defines = dict(re.findall(r"#define\s+(MOE_[A-Z0-9_]+)\s+(-?\d+)", header))
    enums = dict(re.findall(r"\b(MOE_[A-Z0-9_]+)\s*=\s*(-?\d+)", header))
    values = {**enums, **defines}
    checked = 0
    # the shim writes them as tuple assignments: const A, B = Int32(0), Int32(1)
    for names, vals in re.findall(r"^const\s+([A-Z][A-Z0-9_, ]+?)\s*=\s*((?:Int32\(-?\d+\),?\s*)+)$", shim, flags=re.M):
        jnames = [n.strip() for n in names.split(",")]
        jvals = re.findall(r"Int32\((-?\d+)\)", vals)
        assert len(jnames) == len(jvals)
        for jname, jval in zip(jnames, jvals):
            cname = "MOE_" + jname
            assert cname in values, f"{jname} has no {cname} in the header"
            assert int(values[cname]) == int(jval), f"{jname} = {jval} in the shim, {cname} = {values[cname]} in the header"
            checked += 1
    assert checked >= 8, "too few constants of the shim could be matched with the header"

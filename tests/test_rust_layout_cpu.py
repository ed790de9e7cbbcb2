"""The Rust `extern "C"` bindings (rust/ssd-sys/src/lib.rs) against the C header (include/ssd_b200.h): same structs (field
names, order, widths), same constants, same functions (name, argument types in order, return type).  The crate cannot be
compiled here (no cargo / rustc), so this is what keeps the two declarations of the ABI from drifting apart."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "ssd_b200.h")
RUST = os.path.join(ROOT, "rust", "ssd-sys", "src", "lib.rs")

# canonical ABI types: (kind, width in bytes); pointers keep their pointee only as far as the ABI cares (all 8 bytes)
C_TYPES = {"int32_t": "i32", "int64_t": "i64", "size_t": "usize", "float": "f32", "void": "void", "char": "char"}
RUST_TYPES = {"i32": "i32", "i64": "i64", "size_t": "usize", "usize": "usize", "f32": "f32", "c_void": "void", "c_char": "char"}
WIDTH = {"i32": 4, "i64": 8, "usize": 8, "f32": 4, "ptr": 8}


def strip_c_comments(text):
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    return re.sub(r"//[^\n]*", " ", text)


def c_type(decl):
    """'const float*' -> 'ptr'; 'int32_t' -> 'i32'; struct pointers -> 'ptr'."""
    d = decl.replace("const", " ").strip()
    if "*" in d:
        return "ptr"
    d = d.strip()
    return C_TYPES[d]


def parse_header():
    text = strip_c_comments(open(HEADER).read())
    structs = {}
    for body, name in re.findall(r"typedef\s+struct\s+\w+\s*\{(.*?)\}\s*(\w+)\s*;", text, flags=re.S):
        fields = []
        for stmt in body.split(";"):
            stmt = stmt.strip()
            if not stmt:
                continue
            m = re.match(r"(.*?)([\w\s,\*]+)$", stmt, flags=re.S)
            # "int32_t a, b, c" or "const void* x"
            base = re.match(r"((?:const\s+)?\w+)\s*(.*)$", stmt, flags=re.S)
            tname, rest = base.group(1), base.group(2)
            for item in rest.split(","):
                item = item.strip()
                ptr = item.startswith("*") or tname.endswith("*")
                fname = item.lstrip("* ").strip()
                fields.append((fname, "ptr" if ptr or "*" in item else c_type(tname)))
        structs[name] = fields
    funcs = {}
    for ret, name, args in re.findall(r"SSD_API\s+([\w\s\*]+?)\s*\b(ssd_\w+)\s*\((.*?)\)\s*;", text, flags=re.S):
        alist = []
        args = args.strip()
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                if "*" in a:
                    alist.append("ptr")
                else:
                    alist.append(c_type(re.match(r"((?:const\s+)?\w+)", a).group(1)))
        funcs[name] = (c_type(ret) if ret.strip() != "void" else "void", alist)
    consts = {}
    for body in re.findall(r"enum\s*\w*\s*\{(.*?)\}", text, flags=re.S):
        for name, val in re.findall(r"(SSD_\w+)\s*=\s*(-?\d+)", body):
            consts[name] = int(val)
    for name, val in re.findall(r"#define\s+(SSD_\w+)\s+(\d+)\s*$", text, flags=re.M):
        consts[name] = int(val)
    m = re.search(r"#define\s+SSD_NOALLOC_MAX_BYTES\s+\(\(size_t\)(\d+)\s*<<\s*(\d+)\)", text)
    consts["SSD_NOALLOC_MAX_BYTES"] = int(m.group(1)) << int(m.group(2))
    return structs, funcs, consts


def rust_type(t):
    t = t.strip()
    if t.startswith("*const") or t.startswith("*mut"):
        return "ptr"
    return RUST_TYPES[t]


def parse_rust():
    text = re.sub(r"//[^\n]*", " ", open(RUST).read())
    structs = {}
    for name, body in re.findall(r"#\[repr\(C\)\][^\{]*?pub struct (\w+)\s*\{(.*?)\}", text, flags=re.S):
        fields = []
        for fname, ftype in re.findall(r"(?:pub\s+)?(\w+)\s*:\s*([^,\n]+),", body):
            if fname == "_private":
                continue
            fields.append((fname, rust_type(ftype)))
        structs[name] = fields
    funcs = {}
    ext = re.search(r'extern "C"\s*\{(.*)\}', text, flags=re.S).group(1)
    for name, args, ret in re.findall(r"pub fn (ssd_\w+)\s*\((.*?)\)\s*(?:->\s*([^;]+))?;", ext, flags=re.S):
        alist = [rust_type(a.split(":", 1)[1]) for a in args.split(",") if ":" in a]
        funcs[name] = (rust_type(ret) if ret and ret.strip() else "void", alist)
    consts = {}
    for name, val in re.findall(r"pub const (SSD_\w+)\s*:\s*\w+\s*=\s*([^;]+);", text):
        consts[name] = eval(val.strip())
    return structs, funcs, consts


def test_every_struct_has_the_same_fields_in_the_same_order():
    cs, _, _ = parse_header()
    rs, _, _ = parse_rust()
    opaque = {"SsdSpComm"}
    assert set(cs) == set(rs) - opaque, (sorted(cs), sorted(rs))
    for name, fields in cs.items():
        assert fields == rs[name], f"{name}: header {fields} vs Rust {rs[name]}"
        assert sum(WIDTH[t] for _, t in fields) > 0
    assert rs["SsdSpComm"] == []      # opaque handle: no visible field


def test_struct_sizes_equal_the_ctypes_mirror():
    """Third witness: the ctypes structures the GPU tests call through have the size the header's field list implies
    (natural alignment: every 8-byte field of these structs already sits on an 8-byte boundary, except where a lone i32
    precedes a pointer)."""
    import ctypes as C
    from trading_bot_0_b200 import _lib
    cs, _, _ = parse_header()

    def size(fields):
        off = 0
        for _, t in fields:
            w = WIDTH[t]
            off = (off + w - 1) // w * w
            off += w
        return (off + 7) // 8 * 8
    for name in ("SsdDims", "SsdFwdPtrs", "SsdBwdPtrs", "SsdStepDims", "SsdStepPtrs", "SsdConvDims", "SsdConvGrad", "SsdNormDims"):
        assert C.sizeof(getattr(_lib, name)) == size(cs[name]), name


def test_every_function_has_the_same_signature():
    _, cf, _ = parse_header()
    _, rf, _ = parse_rust()
    assert set(cf) == set(rf), (sorted(set(cf) - set(rf)), sorted(set(rf) - set(cf)))
    for name, sig in cf.items():
        assert sig == rf[name], f"{name}: header {sig} vs Rust {rf[name]}"


def test_constants_agree():
    _, _, cc = parse_header()
    _, _, rc = parse_rust()
    for name, val in rc.items():
        assert name in cc, name
        assert cc[name] == val, (name, cc[name], val)
    for needed in ("SSD_OK", "SSD_ERR_TIMEOUT", "SSD_BF16", "SSD_PASS_BWD", "SSD_ALGO_TENSOR_ONETILE", "SSD_STAGE_LOCAL_REST",
                   "SSD_SP_UNIQUE_ID_BYTES", "SSD_NOALLOC_MAX_BYTES"):
        assert needed in rc, needed


def test_build_script_names_every_source_and_the_sm100a_target():
    from trading_bot_0_b200 import build
    text = open(os.path.join(ROOT, "rust", "ssd-sys", "build.rs")).read()
    assert "arch=compute_100a,code=sm_100a" in text
    for src in build.SOURCES:
        assert f'"{src}"' in text, src

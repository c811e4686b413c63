"""Writes ByRE bytecode (MLIR bytecode container version 5, dialect byre_serial 1.0.0) for the tests
of the bytecode reader.  Test infrastructure: the layout follows the one fixture the reference ships
(tests/golden/byre_serial_v1_lljit_case0.mlirbc; MLIR numbers attributes by use count, this writer
by first use, so files differ in order but not in meaning) and, for the attribute and op kinds that
fixture does not contain, the encodings of compiler/lib/Dialect/Byre/IR/Serialization/
Bytecode.cpp:199-330 and ByreSerial.td:355-424.

A module is described as
    {"name": "main", "args": [(argname, argtype, dtype, shape, space), ...],
     "ops": [("alloc", dtype, shape, space) | ("alias", src, offset, dtype, shape, space)
             | ("compute", callee, [operands], {attr: value}, [memory effects] | None)
             | ("copy", src, dst, callee) | ("group_copy", [srcs], [dsts], callee)]}
where operands are value numbers (arguments first, then results in order) and attribute values are
str, bool, int (i64), ("i32", int), float (f32), ("f64", float), ("dense", dtype, shape, [values]),
("array", dtype, [values]), or a list of those.
"""
import numpy as np

SCALAR_KIND = {"i1": 0, "bf16": 1, "f16": 2, "f32": 3, "f64": 4, "index": 10, "i8": 12, "i16": 13, "i32": 14,
               "i64": 15, "ui8": 17, "ui16": 18, "ui32": 19, "ui64": 20}
NP = {"f16": np.float16, "f32": np.float32, "f64": np.float64, "i8": np.int8, "i16": np.int16, "i32": np.int32,
      "i64": np.int64, "ui8": np.uint8, "ui16": np.uint16, "ui32": np.uint32, "ui64": np.uint64}
BITS = {"i1": 1, "i8": 8, "i16": 16, "i32": 32, "i64": 64, "ui8": 8, "ui16": 16, "ui32": 32, "ui64": 64, "index": 64}


def varint(v):
    assert 0 <= v < 1 << 64
    if v < 1 << 7:
        return bytes([(v << 1) | 1])
    for n in range(1, 8):  # n extra bytes carry 7 * (n + 1) bits
        if v < 1 << (7 * (n + 1)):
            return ((v << (n + 1)) | (1 << n)).to_bytes(n + 1, "little")
    return b"\x00" + v.to_bytes(8, "little")


def svarint(v):
    return varint(((v << 1) ^ (v >> 63)) & ((1 << 64) - 1))


def apint(pattern, bits):
    """An integer of known width as MLIR writes it: one byte up to 8 bits, else the zero-extended
    pattern zigzag-coded as a 64-bit signed value."""
    if bits <= 8:
        return bytes([pattern])
    return svarint(pattern - (1 << 64) if pattern >= 1 << 63 else pattern)


def flagged(v, flag):
    return varint((v << 1) | int(flag))


class Writer:
    def __init__(self):
        self.strings, self.attrs, self.types = [], [], []      # interned, in first-use order
        self._s, self._a, self._t = {}, {}, {}

    def string(self, s):
        if s not in self._s:
            self._s[s] = len(self.strings)
            self.strings.append(s)
        return self._s[s]

    def _intern(self, table, index, key, make):
        if key not in index:
            body = make()                 # may intern what it refers to first
            index[key] = len(table)
            table.append(body)
        return index[key]

    # ---- types
    def scalar(self, dt):
        return self._intern(self.types, self._t, ("s", dt), lambda: varint(SCALAR_KIND[dt]))

    def shaped(self, kind, dt, shape, space=None):
        def make():
            elt = self.scalar(dt)
            extra = flagged(self.str_attr(space), 1) if space is not None else varint(0)
            return (varint(kind) + varint(len(shape)) + b"".join(svarint(d) for d in shape) + varint(elt) + extra)
        return self._intern(self.types, self._t, (kind, dt, tuple(shape), space), make)

    def memref(self, dt, shape, space):
        return self.shaped(22, dt, shape, space)

    def tensor(self, dt, shape):
        return self.shaped(23, dt, shape)

    def function(self, inputs):
        return self._intern(self.types, self._t, ("fn", tuple(inputs)),
                            lambda: varint(24) + varint(len(inputs)) + b"".join(varint(t) for t in inputs) + varint(0))

    # ---- attributes
    def raw_attr(self, key, make):
        return self._intern(self.attrs, self._a, key, make)

    def str_attr(self, s):
        return self.raw_attr(("str", s), lambda: varint(5) + varint(self.string(s)))

    def unit(self):
        return self.raw_attr("unit", lambda: varint(2))

    def enum(self, kind, v):
        return self.raw_attr((kind, v), lambda: varint(kind) + varint(v))

    def array(self, items):
        return self.raw_attr(("arr", tuple(items)), lambda: varint(3) + varint(len(items)) + b"".join(varint(i) for i in items))

    def int_attr(self, dt, v):
        def make():
            t = self.scalar(dt)
            bits = BITS[dt]
            pattern = v & ((1 << bits) - 1)
            return varint(0) + varint(t) + apint(pattern, bits)
        return self.raw_attr(("int", dt, v), make)

    def float_attr(self, dt, v):
        def make():
            t = self.scalar(dt)
            pattern = int(np.array(v, NP[dt]).view({"f16": np.uint16, "f32": np.uint32, "f64": np.uint64}[dt]))
            return varint(1) + varint(t) + apint(pattern, {"f16": 16, "f32": 32, "f64": 64}[dt])
        return self.raw_attr(("float", dt, v), make)

    def dense(self, dt, shape, values):
        def make():
            t = self.tensor(dt, shape)
            if dt == "i1":
                vals = [int(bool(v)) for v in values]
                if len(vals) == 1:
                    blob = b"\xff" if vals[0] else b"\x00"
                else:
                    blob = bytes(sum(b << k for k, b in enumerate(vals[i:i + 8])) for i in range(0, len(vals), 8))
            elif dt == "bf16":
                blob = (np.array(values, np.float32).view(np.uint32) >> 16).astype(np.uint16).tobytes()
            else:
                blob = np.array(values, NP[dt]).tobytes()
            return varint(8) + varint(t) + varint(len(blob)) + blob
        return self.raw_attr(("dense", dt, tuple(shape), tuple(values)), make)

    def dense_array(self, dt, values):
        def make():
            t = self.scalar(dt)
            blob = np.array(values, NP[dt]).tobytes()
            return varint(10) + varint(t) + svarint(len(values)) + varint(len(blob)) + blob
        return self.raw_attr(("darr", dt, tuple(values)), make)

    def value(self, v):
        if isinstance(v, str):
            return self.str_attr(v)
        if isinstance(v, bool):
            return self.int_attr("i1", int(v))
        if isinstance(v, int):
            return self.int_attr("i64", v)
        if isinstance(v, float):
            return self.float_attr("f32", v)
        if isinstance(v, list):
            return self.array([self.value(e) for e in v])
        tag = v[0]
        if tag == "dense":
            return self.dense(v[1], v[2], v[3])
        if tag == "array":
            return self.dense_array(v[1], v[2])
        if tag in ("f64", "f16"):
            return self.float_attr(tag, v[1])
        return self.int_attr(tag, v[1])

    def dictionary(self, pairs):
        return self.raw_attr(("dict", tuple(pairs)),
                             lambda: varint(4) + varint(len(pairs)) + b"".join(varint(k) + varint(v) for k, v in pairs))

    def symbol(self, name):
        return self.raw_attr(("sym", name), lambda: varint(7) + varint(self.str_attr(name)) + varint(0))

    def type_attr(self, t):
        return self.raw_attr(("type", t), lambda: varint(6) + varint(t))


def section(sid, body):
    return bytes([sid]) + varint(len(body)) + body


def write_module(desc, producer="MLIR17.0.0git", isolated_func=False):
    """The bytes of one module; strings, attributes and types are numbered in the order of first use."""
    w = Writer()
    used_ops = ["module_v1", "func_v1"]
    for op in desc["ops"]:
        name = {"alloc": "alloc_v1", "alias": "alias", "compute": "compute_v1", "copy": "copy_v1",
                "group_copy": "group_copy_v1"}[op[0]]
        if name not in used_ops:
            used_ops.append(name)
    used_ops.append("return_v1")
    for s in ["byre_serial", "builtin"] + used_ops:
        w.string(s)
    op_id = {n: i for i, n in enumerate(used_ops)}

    arg_types = []
    for (argname, argtype, dt, shape, space) in desc["args"]:
        arg_types.append(w.memref(dt, shape, space))
    argtype_attrs = w.array([w.enum(11, a[1]) for a in desc["args"]])
    names = w.array([w.str_attr(a[0]) for a in desc["args"]])
    fn_type = w.type_attr(w.function(arg_types))
    unit = w.unit()
    module_prop = varint(unit) + varint(0) + varint(0)
    func_prop = (varint(0) + varint(names) + varint(argtype_attrs) + varint(unit) + varint(0) + varint(fn_type) +
                 varint(w.str_attr(desc["name"])) + varint(0) + varint(0))

    n_values = len(desc["args"])
    body_ops = []
    for op in desc["ops"]:
        if op[0] == "alloc":
            _, dt, shape, space = op
            seg = w.dense_array("i32", [0, 0])
            body_ops.append(("alloc_v1", 0x42, varint(0) + varint(seg), (w.memref(dt, shape, space),), ()))
            n_values += 1
        elif op[0] == "alias":
            _, src, offset, dt, shape, space = op
            body_ops.append(("alias", 0x46, varint(w.int_attr("i64", offset)), (w.memref(dt, shape, space),), (src,)))
            n_values += 1
        elif op[0] == "compute":
            _, callee, operands, attrs, effects = op
            prop = varint(w.symbol(callee))
            pairs = [(w.str_attr(k), w.value(v)) for k, v in sorted(attrs.items())]
            prop += flagged(w.dictionary(pairs), 1)
            prop += flagged(w.array([w.enum(12, e) for e in effects]), 1) if effects is not None else varint(0)
            body_ops.append(("compute_v1", 0x44, prop, (), tuple(operands)))
        elif op[0] == "copy":
            _, src, dst, callee = op
            body_ops.append(("copy_v1", 0x44, varint(w.str_attr(callee)), (), (src, dst)))
        elif op[0] == "group_copy":
            _, srcs, dsts, callee = op
            body_ops.append(("group_copy_v1", 0x44, varint(w.str_attr(callee)), (), tuple(srcs) + tuple(dsts)))
    loc = len(w.attrs)  # the builtin unknown location comes last

    # IR section: top-level block, module, its region, func, its region and block, the body
    region = varint(1) + varint(n_values) + varint(((len(body_ops) + 1) << 1) | 1)
    region += varint(len(arg_types)) + b"".join(flagged(t, 0) for t in arg_types) + b"\x00"
    all_props = [module_prop, func_prop]
    for name, mask, prop, results, operands in body_ops:
        region += varint(op_id[name]) + bytes([mask]) + varint(loc) + varint(len(all_props))
        all_props.append(prop)
        if results:
            region += varint(len(results)) + b"".join(varint(t) for t in results)
        if operands:
            region += varint(len(operands)) + b"".join(varint(v) for v in operands)
    region += varint(op_id["return_v1"]) + bytes([0x00]) + varint(loc)
    ir = varint((1 << 1) | 0)
    ir += varint(op_id["module_v1"]) + bytes([0x50]) + varint(loc) + varint(0) + flagged(1, 0)
    ir += varint(1) + varint(0) + varint((1 << 1) | 0)
    ir += varint(op_id["func_v1"]) + bytes([0x50]) + varint(loc) + varint(1)
    # a region marked isolated from above travels in an IR section of its own (lazy loading)
    ir += flagged(1, 1) + section(4, region) if isolated_func else flagged(1, 0) + region

    dialect = (varint(2) + flagged(w.string("byre_serial"), 1) + section(7, varint(0)) + flagged(w.string("builtin"), 0) +
               varint(len(used_ops)) + varint(0) + varint(len(used_ops)) +
               b"".join(flagged(w.string(n), 1) for n in used_ops))
    attr_bodies = w.attrs + [varint(15)]  # builtin UnknownLoc
    offsets = (varint(len(attr_bodies)) + varint(len(w.types)) +
               varint(0) + varint(len(w.attrs)) + b"".join(flagged(len(a), 1) for a in w.attrs) +
               varint(1) + varint(1) + flagged(1, 1) +
               varint(0) + varint(len(w.types)) + b"".join(flagged(len(t), 1) for t in w.types))
    attr_type = b"".join(attr_bodies) + b"".join(w.types)
    strings = (varint(len(w.strings)) + b"".join(varint(len(s.encode()) + 1) for s in reversed(w.strings)) +
               b"".join(s.encode() + b"\x00" for s in w.strings))
    properties = varint(len(all_props)) + b"".join(varint(len(p)) + p for p in all_props)
    return (b"ML\xefR" + varint(5) + producer.encode() + b"\x00" + section(1, dialect) + section(3, offsets) +
            section(2, attr_type) + section(4, ir) + section(6, varint(0)) + section(5, b"") + section(0, strings) +
            section(8, properties))

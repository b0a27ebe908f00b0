"""A small WebAssembly executor: TEST INFRASTRUCTURE ONLY (nothing in the product imports it).

Purpose: run the reference's own shipped kernels, ``src/gpu/wasm-kernels.wasm`` (built from
``rust/wasm-kernels/src/lib.rs``) and ``src/engines/asr-parakeet/parakeet-decoder.wasm`` (built from
``rust/parakeet-decoder/src/lib.rs``), so that the C restatement in this directory can be compared
with outputs of the reference itself, bit for bit.  The host-side calling convention it is driven
with is the one of ``src/gpu/wasm-context.js:135-213`` (``wasm_reset`` / ``wasm_alloc``, copy the
inputs into linear memory, call the kernel with byte pointers, slice the result out).

It executes a module; it prints no listing of it.  Covered: the WebAssembly 1.0 instruction set
(structured control, i32/i64/f32/f64 arithmetic, memory), sign-extension and saturating
truncation, bulk memory copy/fill, and the part of fixed-width SIMD those two modules use.
An instruction outside that set raises ``NotImplementedError`` with its opcode.

f32 arithmetic is done on ``numpy.float32`` scalars and 4-lane ``float32`` arrays, i.e. IEEE-754
binary32 with round-to-nearest-even per operation, which is what WebAssembly specifies (no fused
multiply-add exists in the fixed-width SIMD proposal; ``f32x4.mul`` then ``f32x4.add`` round twice).
"""
from __future__ import annotations

import struct

import numpy as np

PAGE = 65536
M32 = 0xFFFFFFFF
M64 = 0xFFFFFFFFFFFFFFFF
F32 = np.float32
F64 = np.float64

np.seterr(all="ignore")


class Trap(Exception):
    pass


def _s32(x):
    return x - 0x100000000 if x & 0x80000000 else x


def _s64(x):
    return x - (1 << 64) if x & (1 << 63) else x


class _Reader:
    def __init__(self, b, p=0):
        self.b = b
        self.p = p

    def byte(self):
        v = self.b[self.p]
        self.p += 1
        return v

    def u(self):
        r = 0
        s = 0
        while True:
            x = self.b[self.p]
            self.p += 1
            r |= (x & 0x7F) << s
            s += 7
            if not x & 0x80:
                return r

    def s(self):
        r = 0
        s = 0
        while True:
            x = self.b[self.p]
            self.p += 1
            r |= (x & 0x7F) << s
            s += 7
            if not x & 0x80:
                break
        if x & 0x40:
            r -= 1 << s
        return r

    def take(self, n):
        v = self.b[self.p:self.p + n]
        self.p += n
        return v

    def name(self):
        return bytes(self.take(self.u())).decode()


# opcodes whose immediate is one memarg (align, offset)
_MEM_OPS = set(range(0x28, 0x3F))
# SIMD opcodes (0xFD prefix) with a memarg
_SIMD_MEM = set(range(0x00, 0x0C)) | {0x5C, 0x5D}
_SIMD_MEM_LANE = set(range(0x54, 0x5C))
_SIMD_LANE = set(range(0x15, 0x23))


class _Func:
    __slots__ = ("type", "nlocals", "local_types", "code", "nparams", "nresults")


class Module:
    """Decoded module: types, functions, memory limits, globals, exports, data segments."""

    def __init__(self, data: bytes):
        b = bytes(data)
        if b[:8] != b"\0asm\x01\0\0\0":
            raise ValueError("not a WebAssembly 1.0 binary")
        self.types = []
        self.func_types = []
        self.funcs = []
        self.mem_min = 0
        self.mem_max = None
        self.globals = []
        self.exports = {}
        self.datas = []
        self.tables = []
        self.elems = []
        self.start = None
        r = _Reader(b, 8)
        while r.p < len(b):
            sid = r.byte()
            size = r.u()
            end = r.p + size
            if sid == 1:
                for _ in range(r.u()):
                    assert r.byte() == 0x60
                    params = [r.byte() for _ in range(r.u())]
                    results = [r.byte() for _ in range(r.u())]
                    self.types.append((params, results))
            elif sid == 2:
                if r.u() != 0:
                    raise NotImplementedError("imports are not supported (the two reference modules have none)")
            elif sid == 3:
                self.func_types = [r.u() for _ in range(r.u())]
            elif sid == 4:
                for _ in range(r.u()):
                    r.byte()
                    flag = r.byte()
                    mn = r.u()
                    if flag & 1:
                        r.u()
                    self.tables.append([None] * mn)
            elif sid == 5:
                for _ in range(r.u()):
                    flag = r.byte()
                    self.mem_min = r.u()
                    self.mem_max = r.u() if flag & 1 else None
            elif sid == 6:
                for _ in range(r.u()):
                    vt = r.byte()
                    r.byte()  # mutability
                    self.globals.append(self._const_expr(r, vt))
            elif sid == 7:
                for _ in range(r.u()):
                    nm = r.name()
                    kind = r.byte()
                    idx = r.u()
                    self.exports[nm] = (kind, idx)
            elif sid == 8:
                self.start = r.u()
            elif sid == 9:
                for _ in range(r.u()):
                    flag = r.u()
                    if flag != 0:
                        raise NotImplementedError("element segment kind %d" % flag)
                    off = self._const_expr(r, 0x7F)
                    self.elems.append((off, [r.u() for _ in range(r.u())]))
            elif sid == 10:
                n = r.u()
                for i in range(n):
                    bsize = r.u()
                    bend = r.p + bsize
                    f = _Func()
                    f.type = self.types[self.func_types[i]]
                    f.nparams = len(f.type[0])
                    f.nresults = len(f.type[1])
                    lt = list(f.type[0])
                    for _ in range(r.u()):
                        cnt = r.u()
                        t = r.byte()
                        lt.extend([t] * cnt)
                    f.local_types = lt
                    f.nlocals = len(lt)
                    f.code = _decode_body(r, bend, self)
                    assert r.p == bend
                    self.funcs.append(f)
            elif sid == 11:
                for _ in range(r.u()):
                    flag = r.u()
                    if flag == 0:
                        off = self._const_expr(r, 0x7F)
                    elif flag == 1:
                        off = None
                    else:
                        r.u()
                        off = self._const_expr(r, 0x7F)
                    self.datas.append((off, bytes(r.take(r.u()))))
            r.p = end

    @staticmethod
    def _const_expr(r, vt):
        op = r.byte()
        if op == 0x41:
            v = r.s() & M32
        elif op == 0x42:
            v = r.s() & M64
        elif op == 0x43:
            v = F32(struct.unpack("<f", r.take(4))[0])
        elif op == 0x44:
            v = F64(struct.unpack("<d", r.take(8))[0])
        else:
            raise NotImplementedError("constant expression opcode 0x%02x" % op)
        assert r.byte() == 0x0B
        return v


def _blocktype(r, mod):
    """Returns (nparams, nresults) of a block type."""
    b = r.b[r.p]
    if b == 0x40:
        r.p += 1
        return (0, 0)
    if b in (0x7F, 0x7E, 0x7D, 0x7C, 0x7B, 0x70, 0x6F):
        r.p += 1
        return (0, 1)
    t = mod.types[r.s()]
    return (len(t[0]), len(t[1]))


def _decode_body(r, end, mod):
    """Flat instruction list [(opcode, imm...)], with block ends and else targets resolved.

    Opcodes of the 0xFC / 0xFD prefixes are stored as 0xFC00+sub / 0xFD000+sub.
    """
    code = []
    ctl = []  # indices of open block/loop/if
    while r.p < end:
        op = r.byte()
        if op in (0x02, 0x03, 0x04):
            bt = _blocktype(r, mod)
            ctl.append(len(code))
            code.append([op, bt, None, None])  # [op, type, end_pc, else_pc]
        elif op == 0x05:
            code[ctl[-1]][3] = len(code)
            code.append([op, None])  # patched with the end pc below
        elif op == 0x0B:
            if ctl:
                i = ctl.pop()
                code[i][2] = len(code)
                if code[i][3] is not None:
                    code[code[i][3]][1] = len(code)
            code.append([op])
        elif op in (0x0C, 0x0D):
            code.append([op, r.u()])
        elif op == 0x0E:
            tgt = [r.u() for _ in range(r.u())]
            code.append([op, tgt, r.u()])
        elif op in (0x10, 0x20, 0x21, 0x22, 0x23, 0x24):
            code.append([op, r.u()])
        elif op == 0x11:
            code.append([op, r.u(), r.u()])
        elif op in _MEM_OPS:
            r.u()
            code.append([op, r.u()])
        elif op in (0x3F, 0x40):
            r.byte()
            code.append([op])
        elif op == 0x41:
            code.append([op, r.s() & M32])
        elif op == 0x42:
            code.append([op, r.s() & M64])
        elif op == 0x43:
            code.append([op, F32(struct.unpack("<f", r.take(4))[0])])
        elif op == 0x44:
            code.append([op, F64(struct.unpack("<d", r.take(8))[0])])
        elif op == 0x1C:
            for _ in range(r.u()):
                r.byte()
            code.append([0x1B])
        elif op == 0xFC:
            sub = r.u()
            if sub <= 7:
                code.append([0xFC00 + sub])
            elif sub == 8:  # memory.init
                seg = r.u()
                r.byte()
                code.append([0xFC00 + sub, seg])
            elif sub == 9:
                code.append([0xFC00 + sub, r.u()])
            elif sub == 10:
                r.byte()
                r.byte()
                code.append([0xFC00 + sub])
            elif sub == 11:
                r.byte()
                code.append([0xFC00 + sub])
            else:
                raise NotImplementedError("opcode 0xFC %d" % sub)
        elif op == 0xFD:
            sub = r.u()
            if sub in _SIMD_MEM:
                r.u()
                code.append([0xFD000 + sub, r.u()])
            elif sub in _SIMD_MEM_LANE:
                r.u()
                off = r.u()
                code.append([0xFD000 + sub, off, r.byte()])
            elif sub == 0x0C:
                code.append([0xFD000 + sub, bytes(r.take(16))])
            elif sub == 0x0D:
                code.append([0xFD000 + sub, bytes(r.take(16))])
            elif sub in _SIMD_LANE:
                code.append([0xFD000 + sub, r.byte()])
            else:
                code.append([0xFD000 + sub])
        else:
            code.append([op])
    return [tuple(c) for c in code]


def _trunc(x):
    return int(x)  # toward zero


_V_F32 = np.dtype("<f4")
_V_I32 = np.dtype("<i4")
_V_U32 = np.dtype("<u4")
_V_I16 = np.dtype("<i2")
_V_U16 = np.dtype("<u2")
_V_I8 = np.dtype("i1")
_V_U8 = np.dtype("u1")
_V_I64 = np.dtype("<i8")
_V_F64 = np.dtype("<f8")


def _vf(v):
    return np.frombuffer(v, _V_F32)


def _vi(v, dt):
    return np.frombuffer(v, dt)


class Instance:
    """One instantiated module: linear memory, globals, exported functions callable by name."""

    def __init__(self, data: bytes):
        self.mod = m = Module(data)
        self.mem = bytearray(m.mem_min * PAGE)
        self.globals = list(m.globals)
        self.tables = [list(t) for t in m.tables]
        for off, idxs in m.elems:
            self.tables[0][off:off + len(idxs)] = idxs
        for off, d in m.datas:
            if off is not None:
                self.mem[off:off + len(d)] = d
        self.steps = 0
        if m.start is not None:
            self._call(m.start, [])

    # ---- host-side helpers -------------------------------------------------------------
    def export_names(self, kind=0):
        return sorted(k for k, (kd, _) in self.mod.exports.items() if kd == kind)

    def global_value(self, name):
        kind, idx = self.mod.exports[name]
        assert kind == 3
        return self.globals[idx]

    def call(self, name, *args):
        kind, idx = self.mod.exports[name]
        assert kind == 0, name
        f = self.mod.funcs[idx]
        vals = []
        for a, t in zip(args, f.type[0]):
            if t == 0x7F:
                vals.append(int(a) & M32)
            elif t == 0x7E:
                vals.append(int(a) & M64)
            elif t == 0x7D:
                vals.append(F32(a))
            else:
                vals.append(F64(a))
        assert len(vals) == f.nparams, (name, len(vals), f.nparams)
        res = self._call(idx, vals)
        if not res:
            return None
        return res[0] if len(res) == 1 else tuple(res)

    def write(self, ptr, arr):
        b = np.ascontiguousarray(arr).tobytes()
        if ptr + len(b) > len(self.mem):
            raise Trap("host write out of bounds")
        self.mem[ptr:ptr + len(b)] = b

    def read(self, ptr, count, dtype):
        dt = np.dtype(dtype)
        return np.frombuffer(bytes(self.mem[ptr:ptr + count * dt.itemsize]), dt).copy()

    # ---- execution ------------------------------------------------------------------------
    def _call(self, fidx, args):
        f = self.mod.funcs[fidx]
        locs = list(args)
        for t in f.local_types[f.nparams:]:
            locs.append(0 if t in (0x7F, 0x7E) else F32(0) if t == 0x7D else F64(0) if t == 0x7C else bytes(16))
        return self._run(f, locs)

    def _run(self, f, locs):  # noqa: C901 - one flat dispatch loop on purpose
        code = f.code
        st = []
        push = st.append
        pop = st.pop
        # label stack entries: (continuation pc, arity, stack height)
        labels = [(len(code), f.nresults, 0)]
        pc = 0
        n = len(code)
        mem = self.mem
        up = struct.unpack_from
        pk = struct.pack_into
        steps = 0
        while pc < n:
            ins = code[pc]
            op = ins[0]
            pc += 1
            steps += 1
            # --- hottest first -------------------------------------------------------------
            if op == 0x20:
                push(locs[ins[1]])
            elif op == 0x21:
                locs[ins[1]] = pop()
            elif op == 0x22:
                locs[ins[1]] = st[-1]
            elif op == 0x41 or op == 0x42 or op == 0x43 or op == 0x44:
                push(ins[1])
            elif op == 0x6A:
                b = pop()
                st[-1] = (st[-1] + b) & M32
            elif op == 0x6B:
                b = pop()
                st[-1] = (st[-1] - b) & M32
            elif op == 0x6C:
                b = pop()
                st[-1] = (st[-1] * b) & M32
            elif op == 0x92:
                b = pop()
                st[-1] = st[-1] + b
            elif op == 0x94:
                b = pop()
                st[-1] = st[-1] * b
            elif op == 0x93:
                b = pop()
                st[-1] = st[-1] - b
            elif op == 0x2A:
                a = st[-1] + ins[1]
                if a + 4 > len(mem):
                    raise Trap("out of bounds memory access")
                st[-1] = F32(up("<f", mem, a)[0])
            elif op == 0x38:
                v = pop()
                a = pop() + ins[1]
                if a + 4 > len(mem):
                    raise Trap("out of bounds memory access")
                pk("<f", mem, a, v)
            elif op == 0x28:
                a = st[-1] + ins[1]
                if a + 4 > len(mem):
                    raise Trap("out of bounds memory access")
                st[-1] = up("<I", mem, a)[0]
            elif op == 0x36:
                v = pop()
                a = pop() + ins[1]
                if a + 4 > len(mem):
                    raise Trap("out of bounds memory access")
                pk("<I", mem, a, v)
            elif op == 0x2C:
                a = st[-1] + ins[1]
                if a + 1 > len(mem):
                    raise Trap("out of bounds memory access")
                v = mem[a]
                st[-1] = (v - 256) & M32 if v & 0x80 else v
            elif op == 0x2D:
                a = st[-1] + ins[1]
                if a + 1 > len(mem):
                    raise Trap("out of bounds memory access")
                st[-1] = mem[a]
            elif op == 0x0D:
                if pop():
                    pc = self._branch(ins[1], labels, st)
            elif op == 0x0C:
                pc = self._branch(ins[1], labels, st)
            elif op == 0x02:
                labels.append((ins[2] + 1, ins[1][1], len(st) - ins[1][0]))
            elif op == 0x03:
                labels.append((pc - 1, ins[1][0], len(st) - ins[1][0]))
            elif op == 0x04:
                c = pop()
                if c:
                    labels.append((ins[2] + 1, ins[1][1], len(st) - ins[1][0]))
                elif ins[3] is not None:
                    labels.append((ins[2] + 1, ins[1][1], len(st) - ins[1][0]))
                    pc = ins[3] + 1
                else:
                    pc = ins[2] + 1
            elif op == 0x05:
                # reached the end of the then-arm: leave the block
                labels.pop()
                pc = ins[1] + 1
            elif op == 0x0B:
                if pc < n or len(labels) > 1:
                    labels.pop()
            # --- comparisons ------------------------------------------------------------------
            elif op == 0x45 or op == 0x50:
                st[-1] = 1 if st[-1] == 0 else 0
            elif op == 0x46 or op == 0x51:
                b = pop()
                st[-1] = 1 if st[-1] == b else 0
            elif op == 0x47 or op == 0x52:
                b = pop()
                st[-1] = 1 if st[-1] != b else 0
            elif op == 0x48:
                b = pop()
                st[-1] = 1 if _s32(st[-1]) < _s32(b) else 0
            elif op == 0x49 or op == 0x54:
                b = pop()
                st[-1] = 1 if st[-1] < b else 0
            elif op == 0x4A:
                b = pop()
                st[-1] = 1 if _s32(st[-1]) > _s32(b) else 0
            elif op == 0x4B or op == 0x56:
                b = pop()
                st[-1] = 1 if st[-1] > b else 0
            elif op == 0x4C:
                b = pop()
                st[-1] = 1 if _s32(st[-1]) <= _s32(b) else 0
            elif op == 0x4D or op == 0x58:
                b = pop()
                st[-1] = 1 if st[-1] <= b else 0
            elif op == 0x4E:
                b = pop()
                st[-1] = 1 if _s32(st[-1]) >= _s32(b) else 0
            elif op == 0x4F or op == 0x5A:
                b = pop()
                st[-1] = 1 if st[-1] >= b else 0
            elif op == 0x53:
                b = pop()
                st[-1] = 1 if _s64(st[-1]) < _s64(b) else 0
            elif op == 0x55:
                b = pop()
                st[-1] = 1 if _s64(st[-1]) > _s64(b) else 0
            elif op == 0x57:
                b = pop()
                st[-1] = 1 if _s64(st[-1]) <= _s64(b) else 0
            elif op == 0x59:
                b = pop()
                st[-1] = 1 if _s64(st[-1]) >= _s64(b) else 0
            elif op == 0x5B or op == 0x61:
                b = pop()
                st[-1] = 1 if st[-1] == b else 0
            elif op == 0x5C or op == 0x62:
                b = pop()
                st[-1] = 1 if st[-1] != b else 0
            elif op == 0x5D or op == 0x63:
                b = pop()
                st[-1] = 1 if st[-1] < b else 0
            elif op == 0x5E or op == 0x64:
                b = pop()
                st[-1] = 1 if st[-1] > b else 0
            elif op == 0x5F or op == 0x65:
                b = pop()
                st[-1] = 1 if st[-1] <= b else 0
            elif op == 0x60 or op == 0x66:
                b = pop()
                st[-1] = 1 if st[-1] >= b else 0
            # --- i32 arithmetic -----------------------------------------------------------------
            elif op == 0x67:
                v = st[-1]
                st[-1] = 32 - v.bit_length()
            elif op == 0x68:
                v = st[-1]
                st[-1] = 32 if v == 0 else (v & -v).bit_length() - 1
            elif op == 0x69:
                st[-1] = bin(st[-1]).count("1")
            elif op == 0x6D:
                b = _s32(pop())
                a = _s32(st[-1])
                if b == 0:
                    raise Trap("integer divide by zero")
                q = abs(a) // abs(b)
                st[-1] = (q if (a < 0) == (b < 0) else -q) & M32
            elif op == 0x6E:
                b = pop()
                if b == 0:
                    raise Trap("integer divide by zero")
                st[-1] = st[-1] // b
            elif op == 0x6F:
                b = _s32(pop())
                a = _s32(st[-1])
                if b == 0:
                    raise Trap("integer divide by zero")
                r_ = abs(a) % abs(b)
                st[-1] = (-r_ if a < 0 else r_) & M32
            elif op == 0x70:
                b = pop()
                if b == 0:
                    raise Trap("integer divide by zero")
                st[-1] = st[-1] % b
            elif op == 0x71 or op == 0x83:
                b = pop()
                st[-1] = st[-1] & b
            elif op == 0x72 or op == 0x84:
                b = pop()
                st[-1] = st[-1] | b
            elif op == 0x73 or op == 0x85:
                b = pop()
                st[-1] = st[-1] ^ b
            elif op == 0x74:
                b = pop() & 31
                st[-1] = (st[-1] << b) & M32
            elif op == 0x75:
                b = pop() & 31
                st[-1] = (_s32(st[-1]) >> b) & M32
            elif op == 0x76:
                b = pop() & 31
                st[-1] = st[-1] >> b
            elif op == 0x77:
                b = pop() & 31
                a = st[-1]
                st[-1] = ((a << b) | (a >> (32 - b))) & M32
            elif op == 0x78:
                b = pop() & 31
                a = st[-1]
                st[-1] = ((a >> b) | (a << (32 - b))) & M32
            # --- i64 arithmetic -----------------------------------------------------------------
            elif op == 0x79:
                st[-1] = 64 - st[-1].bit_length()
            elif op == 0x7A:
                v = st[-1]
                st[-1] = 64 if v == 0 else (v & -v).bit_length() - 1
            elif op == 0x7B:
                st[-1] = bin(st[-1]).count("1")
            elif op == 0x7C:
                b = pop()
                st[-1] = (st[-1] + b) & M64
            elif op == 0x7D:
                b = pop()
                st[-1] = (st[-1] - b) & M64
            elif op == 0x7E:
                b = pop()
                st[-1] = (st[-1] * b) & M64
            elif op == 0x7F:
                b = _s64(pop())
                a = _s64(st[-1])
                if b == 0:
                    raise Trap("integer divide by zero")
                q = abs(a) // abs(b)
                st[-1] = (q if (a < 0) == (b < 0) else -q) & M64
            elif op == 0x80:
                b = pop()
                if b == 0:
                    raise Trap("integer divide by zero")
                st[-1] = st[-1] // b
            elif op == 0x81:
                b = _s64(pop())
                a = _s64(st[-1])
                if b == 0:
                    raise Trap("integer divide by zero")
                r_ = abs(a) % abs(b)
                st[-1] = (-r_ if a < 0 else r_) & M64
            elif op == 0x82:
                b = pop()
                if b == 0:
                    raise Trap("integer divide by zero")
                st[-1] = st[-1] % b
            elif op == 0x86:
                b = pop() & 63
                st[-1] = (st[-1] << b) & M64
            elif op == 0x87:
                b = pop() & 63
                st[-1] = (_s64(st[-1]) >> b) & M64
            elif op == 0x88:
                b = pop() & 63
                st[-1] = st[-1] >> b
            elif op == 0x89:
                b = pop() & 63
                a = st[-1]
                st[-1] = ((a << b) | (a >> (64 - b))) & M64
            elif op == 0x8A:
                b = pop() & 63
                a = st[-1]
                st[-1] = ((a >> b) | (a << (64 - b))) & M64
            # --- float arithmetic (numpy scalars keep the width) -----------------------------------
            elif op == 0x8B or op == 0x99:
                st[-1] = abs(st[-1])
            elif op == 0x8C or op == 0x9A:
                st[-1] = -st[-1]
            elif op == 0x8D or op == 0x9B:
                st[-1] = np.ceil(st[-1])
            elif op == 0x8E or op == 0x9C:
                st[-1] = np.floor(st[-1])
            elif op == 0x8F or op == 0x9D:
                st[-1] = np.trunc(st[-1])
            elif op == 0x90 or op == 0x9E:
                st[-1] = np.rint(st[-1])
            elif op == 0x91 or op == 0x9F:
                st[-1] = np.sqrt(st[-1])
            elif op == 0x95 or op == 0xA3:
                b = pop()
                st[-1] = st[-1] / b
            elif op == 0x96 or op == 0xA4:
                b = pop()
                a = st[-1]
                st[-1] = a + b if (a != a or b != b) else (np.minimum(a, b) if a != b else (a if np.signbit(a) else b))
            elif op == 0x97 or op == 0xA5:
                b = pop()
                a = st[-1]
                st[-1] = a + b if (a != a or b != b) else (np.maximum(a, b) if a != b else (b if np.signbit(a) else a))
            elif op == 0x98 or op == 0xA6:
                b = pop()
                st[-1] = np.copysign(st[-1], b)
            elif op == 0xA0:
                b = pop()
                st[-1] = st[-1] + b
            elif op == 0xA1:
                b = pop()
                st[-1] = st[-1] - b
            elif op == 0xA2:
                b = pop()
                st[-1] = st[-1] * b
            # --- conversions ------------------------------------------------------------------------
            elif op == 0xA7:
                st[-1] = st[-1] & M32
            elif op == 0xA8 or op == 0xAA:
                v = st[-1]
                if v != v or not (-2147483649.0 < float(v) < 2147483648.0):
                    raise Trap("invalid conversion to integer")
                st[-1] = _trunc(v) & M32
            elif op == 0xA9 or op == 0xAB:
                v = st[-1]
                if v != v or not (-1.0 < float(v) < 4294967296.0):
                    raise Trap("invalid conversion to integer")
                st[-1] = _trunc(v) & M32
            elif op == 0xAC:
                st[-1] = _s32(st[-1]) & M64
            elif op == 0xAD:
                pass
            elif op == 0xAE or op == 0xB0:
                v = st[-1]
                if v != v or not (-9223372036854777856.0 < float(v) < 9223372036854775808.0):
                    raise Trap("invalid conversion to integer")
                st[-1] = _trunc(v) & M64
            elif op == 0xAF or op == 0xB1:
                v = st[-1]
                if v != v or not (-1.0 < float(v) < 18446744073709551616.0):
                    raise Trap("invalid conversion to integer")
                st[-1] = _trunc(v) & M64
            elif op == 0xB2:
                st[-1] = F32(_s32(st[-1]))
            elif op == 0xB3:
                st[-1] = F32(st[-1])
            elif op == 0xB4:
                st[-1] = F32(np.int64(_s64(st[-1])))
            elif op == 0xB5:
                st[-1] = F32(np.uint64(st[-1]))
            elif op == 0xB6:
                st[-1] = F32(st[-1])
            elif op == 0xB7:
                st[-1] = F64(_s32(st[-1]))
            elif op == 0xB8:
                st[-1] = F64(st[-1])
            elif op == 0xB9:
                st[-1] = F64(np.int64(_s64(st[-1])))
            elif op == 0xBA:
                st[-1] = F64(np.uint64(st[-1]))
            elif op == 0xBB:
                st[-1] = F64(st[-1])
            elif op == 0xBC:
                st[-1] = struct.unpack("<I", struct.pack("<f", st[-1]))[0]
            elif op == 0xBD:
                st[-1] = struct.unpack("<Q", struct.pack("<d", st[-1]))[0]
            elif op == 0xBE:
                st[-1] = F32(struct.unpack("<f", struct.pack("<I", st[-1]))[0])
            elif op == 0xBF:
                st[-1] = F64(struct.unpack("<d", struct.pack("<Q", st[-1]))[0])
            elif op == 0xC0:
                v = st[-1] & 0xFF
                st[-1] = (v - 256) & M32 if v & 0x80 else v
            elif op == 0xC1:
                v = st[-1] & 0xFFFF
                st[-1] = (v - 65536) & M32 if v & 0x8000 else v
            elif op == 0xC2:
                v = st[-1] & 0xFF
                st[-1] = (v - 256) & M64 if v & 0x80 else v
            elif op == 0xC3:
                v = st[-1] & 0xFFFF
                st[-1] = (v - 65536) & M64 if v & 0x8000 else v
            elif op == 0xC4:
                st[-1] = _s32(st[-1] & M32) & M64
            # --- parametric / variable / control ------------------------------------------------------
            elif op == 0x1A:
                pop()
            elif op == 0x1B:
                c = pop()
                b = pop()
                if not c:
                    st[-1] = b
            elif op == 0x23:
                push(self.globals[ins[1]])
            elif op == 0x24:
                self.globals[ins[1]] = pop()
            elif op == 0x00:
                raise Trap("unreachable")
            elif op == 0x01:
                pass
            elif op == 0x0E:
                i = pop()
                tg = ins[1]
                pc = self._branch(tg[i] if i < len(tg) else ins[2], labels, st)
            elif op == 0x0F:
                pc = self._branch(len(labels) - 1, labels, st)
            elif op == 0x10:
                g = self.mod.funcs[ins[1]]
                k = g.nparams
                args = st[len(st) - k:] if k else []
                if k:
                    del st[len(st) - k:]
                self.steps += steps
                steps = 0
                st.extend(self._call(ins[1], args))
                mem = self.mem
            elif op == 0x11:
                i = pop()
                tbl = self.tables[ins[2]]
                if i >= len(tbl) or tbl[i] is None:
                    raise Trap("undefined table element")
                fi = tbl[i]
                g = self.mod.funcs[fi]
                if g.type != self.mod.types[ins[1]]:
                    raise Trap("indirect call type mismatch")
                k = g.nparams
                args = st[len(st) - k:] if k else []
                if k:
                    del st[len(st) - k:]
                st.extend(self._call(fi, args))
                mem = self.mem
            # --- remaining memory ops -----------------------------------------------------------------------
            elif 0x29 <= op <= 0x35:
                a = st[-1] + ins[1]
                fmt, size = _LOADS[op]
                if a + size > len(mem):
                    raise Trap("out of bounds memory access")
                v = up(fmt, mem, a)[0]
                if op == 0x2B:
                    v = F64(v)
                elif op in (0x2E, 0x2F):
                    v &= M32
                elif op != 0x29 and op >= 0x30:
                    v &= M64
                st[-1] = v
            elif 0x37 <= op <= 0x3E:
                v = pop()
                a = pop() + ins[1]
                fmt, size, mask = _STORES[op]
                if a + size > len(mem):
                    raise Trap("out of bounds memory access")
                pk(fmt, mem, a, v & mask if mask else v)
            elif op == 0x3F:
                push(len(mem) // PAGE)
            elif op == 0x40:
                d = pop()
                old = len(mem) // PAGE
                lim = self.mod.mem_max if self.mod.mem_max is not None else 65536
                if old + d > lim:
                    push(M32)
                else:
                    mem.extend(bytes(d * PAGE))
                    push(old)
            elif op == 0xFC0A:
                cnt = pop()
                s = pop()
                d = pop()
                if s + cnt > len(mem) or d + cnt > len(mem):
                    raise Trap("out of bounds memory access")
                mem[d:d + cnt] = mem[s:s + cnt]
            elif op == 0xFC0B:
                cnt = pop()
                val = pop() & 0xFF
                d = pop()
                if d + cnt > len(mem):
                    raise Trap("out of bounds memory access")
                mem[d:d + cnt] = bytes([val]) * cnt
            elif 0xFC00 <= op <= 0xFC07:
                v = st[-1]
                sub = op - 0xFC00
                bits, signed = (32, sub % 2 == 0) if sub < 4 else (64, sub % 2 == 0)
                if v != v:
                    r_ = 0
                else:
                    lo, hi = (-(1 << (bits - 1)), (1 << (bits - 1)) - 1) if signed else (0, (1 << bits) - 1)
                    fv = float(v)
                    r_ = lo if fv <= lo else hi if fv >= hi else _trunc(v)
                st[-1] = r_ & ((1 << bits) - 1)
            elif op >= 0xFD000:
                self._simd(op - 0xFD000, ins, st, mem)
            else:
                raise NotImplementedError("opcode 0x%x" % op)
        self.steps += steps
        k = f.nresults
        return st[len(st) - k:] if k else []

    @staticmethod
    def _branch(depth, labels, st):
        idx = len(labels) - 1 - depth
        cont, arity, height = labels[idx]
        if arity:
            vals = st[len(st) - arity:]
            del st[height:]
            st.extend(vals)
        else:
            del st[height:]
        # a loop label continues at the loop instruction itself (which re-pushes it)
        del labels[idx:]
        return cont

    def _simd(self, sub, ins, st, mem):  # noqa: C901
        pop = st.pop
        if sub == 0x00:  # v128.load
            a = st[-1] + ins[1]
            if a + 16 > len(mem):
                raise Trap("out of bounds memory access")
            st[-1] = bytes(mem[a:a + 16])
        elif sub == 0x0B:  # v128.store
            v = pop()
            a = pop() + ins[1]
            if a + 16 > len(mem):
                raise Trap("out of bounds memory access")
            mem[a:a + 16] = v
        elif 0x01 <= sub <= 0x06:  # load 8x8 / 16x4 / 32x2 extending
            a = st[-1] + ins[1]
            if a + 8 > len(mem):
                raise Trap("out of bounds memory access")
            src, dst = {1: (_V_I8, _V_I16), 2: (_V_U8, _V_U16), 3: (_V_I16, _V_I32), 4: (_V_U16, _V_U32),
                        5: (_V_I32, _V_I64), 6: (np.dtype("<u4"), np.dtype("<u8"))}[sub]
            st[-1] = np.frombuffer(bytes(mem[a:a + 8]), src).astype(dst).tobytes()
        elif 0x07 <= sub <= 0x0A:  # load splat
            size = 1 << (sub - 7)
            a = st[-1] + ins[1]
            if a + size > len(mem):
                raise Trap("out of bounds memory access")
            st[-1] = bytes(mem[a:a + size]) * (16 // size)
        elif sub == 0x5C or sub == 0x5D:  # load32_zero / load64_zero
            size = 4 if sub == 0x5C else 8
            a = st[-1] + ins[1]
            if a + size > len(mem):
                raise Trap("out of bounds memory access")
            st[-1] = bytes(mem[a:a + size]) + bytes(16 - size)
        elif 0x54 <= sub <= 0x57:  # load lane
            size = 1 << (sub - 0x54)
            v = bytearray(pop())
            a = st[-1] + ins[1]
            if a + size > len(mem):
                raise Trap("out of bounds memory access")
            v[ins[2] * size:(ins[2] + 1) * size] = mem[a:a + size]
            st[-1] = bytes(v)
        elif 0x58 <= sub <= 0x5B:  # store lane
            size = 1 << (sub - 0x58)
            v = pop()
            a = pop() + ins[1]
            if a + size > len(mem):
                raise Trap("out of bounds memory access")
            mem[a:a + size] = v[ins[2] * size:(ins[2] + 1) * size]
        elif sub == 0x0C:
            st.append(ins[1])
        elif sub == 0x0D:  # i8x16.shuffle
            b = pop()
            ab = st[-1] + b
            st[-1] = bytes(ab[i] for i in ins[1])
        elif sub == 0x0E:  # i8x16.swizzle
            s = pop()
            a = st[-1]
            st[-1] = bytes(a[i] if i < 16 else 0 for i in s)
        elif sub == 0x0F:
            st[-1] = bytes([st[-1] & 0xFF]) * 16
        elif sub == 0x10:
            st[-1] = struct.pack("<H", st[-1] & 0xFFFF) * 8
        elif sub == 0x11:
            st[-1] = struct.pack("<I", st[-1]) * 4
        elif sub == 0x12:
            st[-1] = struct.pack("<Q", st[-1]) * 2
        elif sub == 0x13:
            st[-1] = struct.pack("<f", st[-1]) * 4
        elif sub == 0x14:
            st[-1] = struct.pack("<d", st[-1]) * 2
        elif sub == 0x15:
            st[-1] = struct.unpack_from("<b", st[-1], ins[1])[0] & M32
        elif sub == 0x16:
            st[-1] = st[-1][ins[1]]
        elif sub == 0x18:
            st[-1] = struct.unpack_from("<h", st[-1], 2 * ins[1])[0] & M32
        elif sub == 0x19:
            st[-1] = struct.unpack_from("<H", st[-1], 2 * ins[1])[0]
        elif sub == 0x1B:
            st[-1] = struct.unpack_from("<I", st[-1], 4 * ins[1])[0]
        elif sub == 0x1D:
            st[-1] = struct.unpack_from("<Q", st[-1], 8 * ins[1])[0]
        elif sub == 0x1F:
            st[-1] = F32(struct.unpack_from("<f", st[-1], 4 * ins[1])[0])
        elif sub == 0x21:
            st[-1] = F64(struct.unpack_from("<d", st[-1], 8 * ins[1])[0])
        elif sub in (0x17, 0x1A, 0x1C, 0x1E, 0x20, 0x22):  # replace_lane
            x = pop()
            v = bytearray(st[-1])
            fmt = {0x17: "<B", 0x1A: "<H", 0x1C: "<I", 0x1E: "<Q", 0x20: "<f", 0x22: "<d"}[sub]
            if sub == 0x17:
                x &= 0xFF
            elif sub == 0x1A:
                x &= 0xFFFF
            struct.pack_into(fmt, v, struct.calcsize(fmt) * ins[1], x)
            st[-1] = bytes(v)
        # f32x4 arithmetic
        elif sub == 0xE4:
            b = pop()
            st[-1] = (_vf(st[-1]) + _vf(b)).tobytes()
        elif sub == 0xE5:
            b = pop()
            st[-1] = (_vf(st[-1]) - _vf(b)).tobytes()
        elif sub == 0xE6:
            b = pop()
            st[-1] = (_vf(st[-1]) * _vf(b)).tobytes()
        elif sub == 0xE7:
            b = pop()
            st[-1] = (_vf(st[-1]) / _vf(b)).tobytes()
        elif sub == 0xE0:
            st[-1] = np.abs(_vf(st[-1])).tobytes()
        elif sub == 0xE1:
            st[-1] = (-_vf(st[-1])).tobytes()
        elif sub == 0xE3:
            st[-1] = np.sqrt(_vf(st[-1])).tobytes()
        elif sub == 0xE8 or sub == 0xE9:  # f32x4.min / max (NaN-propagating, -0 < +0)
            b = _vf(pop())
            a = _vf(st[-1])
            r_ = np.minimum(a, b) if sub == 0xE8 else np.maximum(a, b)
            eq = (a == b)
            if eq.any():
                sa = np.signbit(a)
                pick_a = sa if sub == 0xE8 else ~sa
                r_ = np.where(eq, np.where(pick_a, a, b), r_)
            st[-1] = r_.astype(_V_F32).tobytes()
        elif sub == 0xEA or sub == 0xEB:  # f32x4.pmin / pmax
            b = _vf(pop())
            a = _vf(st[-1])
            st[-1] = (np.where(b < a, b, a) if sub == 0xEA else np.where(a < b, b, a)).astype(_V_F32).tobytes()
        # f32x4 comparisons
        elif 0x41 <= sub <= 0x46:
            b = _vf(pop())
            a = _vf(st[-1])
            m = {0x41: a == b, 0x42: a != b, 0x43: a < b, 0x44: a > b, 0x45: a <= b, 0x46: a >= b}[sub]
            st[-1] = np.where(m, np.uint32(M32), np.uint32(0)).astype(_V_U32).tobytes()
        # bitwise
        elif sub == 0x4D:
            st[-1] = (~_vi(st[-1], _V_U32)).tobytes()
        elif sub == 0x4E:
            b = pop()
            st[-1] = (_vi(st[-1], _V_U32) & _vi(b, _V_U32)).tobytes()
        elif sub == 0x4F:
            b = pop()
            st[-1] = (_vi(st[-1], _V_U32) & ~_vi(b, _V_U32)).tobytes()
        elif sub == 0x50:
            b = pop()
            st[-1] = (_vi(st[-1], _V_U32) | _vi(b, _V_U32)).tobytes()
        elif sub == 0x51:
            b = pop()
            st[-1] = (_vi(st[-1], _V_U32) ^ _vi(b, _V_U32)).tobytes()
        elif sub == 0x52:  # bitselect
            c = _vi(pop(), _V_U32)
            b = _vi(pop(), _V_U32)
            a = _vi(st[-1], _V_U32)
            st[-1] = ((a & c) | (b & ~c)).tobytes()
        elif sub == 0x53:
            st[-1] = 1 if any(st[-1]) else 0
        # integer lane-wise ops, by lane width
        elif sub in _INT_BIN:
            dt, fn = _INT_BIN[sub]
            b = _vi(pop(), dt)
            st[-1] = fn(_vi(st[-1], dt), b).astype(dt).tobytes()
        elif sub in _INT_SHIFT:
            dt, kind = _INT_SHIFT[sub]
            sh = pop() % (dt.itemsize * 8)
            a = _vi(st[-1], dt)
            st[-1] = (a << dt.type(sh) if kind == "l" else a >> dt.type(sh)).astype(dt).tobytes()
        elif sub in _INT_EXTEND:
            src, dst, high = _INT_EXTEND[sub]
            a = _vi(st[-1], src)
            half = len(a) // 2
            st[-1] = (a[half:] if high else a[:half]).astype(dst).tobytes()
        elif sub in _INT_NARROW:
            src, dst = _INT_NARROW[sub]
            b = _vi(pop(), src)
            a = _vi(st[-1], src)
            info = np.iinfo(dst)
            st[-1] = np.clip(np.concatenate([a, b]).astype(np.int64), info.min, info.max).astype(dst).tobytes()
        elif sub == 0xFA:  # f32x4.convert_i32x4_s
            st[-1] = _vi(st[-1], _V_I32).astype(_V_F32).tobytes()
        elif sub == 0xFB:
            st[-1] = _vi(st[-1], _V_U32).astype(_V_F32).tobytes()
        elif sub == 0xF8 or sub == 0xF9:  # i32x4.trunc_sat_f32x4_s / u
            a = _vf(st[-1]).astype(np.float64)
            a = np.where(a != a, 0.0, np.trunc(a))
            if sub == 0xF8:
                st[-1] = np.clip(a, -2147483648.0, 2147483647.0).astype(np.int64).astype(_V_I32).tobytes()
            else:
                st[-1] = np.clip(a, 0.0, 4294967295.0).astype(np.int64).astype(_V_U32).tobytes()
        elif sub == 0xBA:  # i32x4.dot_i16x8_s
            b = _vi(pop(), _V_I16).astype(np.int32)
            a = _vi(st[-1], _V_I16).astype(np.int32)
            p = a * b
            st[-1] = (p[0::2] + p[1::2]).astype(_V_I32).tobytes()
        elif sub in (0x61, 0x81, 0xA1, 0xC1):  # neg
            dt = {0x61: _V_I8, 0x81: _V_I16, 0xA1: _V_I32, 0xC1: _V_I64}[sub]
            st[-1] = (-_vi(st[-1], dt)).astype(dt).tobytes()
        elif sub in (0x60, 0x80, 0xA0, 0xC0):  # abs
            dt = {0x60: _V_I8, 0x80: _V_I16, 0xA0: _V_I32, 0xC0: _V_I64}[sub]
            st[-1] = np.abs(_vi(st[-1], dt)).astype(dt).tobytes()
        elif sub in (0x63, 0x83, 0xA3, 0xC3):  # all_true
            dt = {0x63: _V_I8, 0x83: _V_I16, 0xA3: _V_I32, 0xC3: _V_I64}[sub]
            st[-1] = 1 if _vi(st[-1], dt).all() else 0
        elif sub in (0x64, 0x84, 0xA4, 0xC4):  # bitmask
            dt = {0x64: _V_I8, 0x84: _V_I16, 0xA4: _V_I32, 0xC4: _V_I64}[sub]
            a = _vi(st[-1], dt)
            st[-1] = sum(1 << i for i, x in enumerate(a) if x < 0)
        elif sub in _INT_CMP:
            dt, fn = _INT_CMP[sub]
            b = _vi(pop(), dt)
            a = _vi(st[-1], dt)
            udt = np.dtype("<u%d" % dt.itemsize)
            st[-1] = np.where(fn(a, b), udt.type(-1 & ((1 << (8 * dt.itemsize)) - 1)), udt.type(0)).astype(udt).tobytes()
        else:
            raise NotImplementedError("SIMD opcode 0xFD 0x%x" % sub)


_LOADS = {0x29: ("<Q", 8), 0x2A: ("<f", 4), 0x2B: ("<d", 8), 0x2C: ("<b", 1), 0x2D: ("<B", 1), 0x2E: ("<h", 2),
          0x2F: ("<H", 2), 0x30: ("<b", 1), 0x31: ("<B", 1), 0x32: ("<h", 2), 0x33: ("<H", 2), 0x34: ("<i", 4),
          0x35: ("<I", 4)}
_STORES = {0x37: ("<Q", 8, 0), 0x38: ("<f", 4, 0), 0x39: ("<d", 8, 0), 0x3A: ("<B", 1, 0xFF), 0x3B: ("<H", 2, 0xFFFF),
           0x3C: ("<B", 1, 0xFF), 0x3D: ("<H", 2, 0xFFFF), 0x3E: ("<I", 4, M32)}


def _sat(dt):
    info = np.iinfo(dt)

    def add(a, b):
        return np.clip(a.astype(np.int64) + b.astype(np.int64), info.min, info.max)

    def sub(a, b):
        return np.clip(a.astype(np.int64) - b.astype(np.int64), info.min, info.max)

    return add, sub


_INT_BIN = {}
for _base, _sd, _ud in ((0x6E, _V_I8, _V_U8), (0x8E, _V_I16, _V_U16)):
    _as, _ss = _sat(_sd)
    _au, _su = _sat(_ud)
    _INT_BIN[_base] = (_sd, lambda a, b: a + b)
    _INT_BIN[_base + 1] = (_sd, _as)
    _INT_BIN[_base + 2] = (_ud, _au)
    _INT_BIN[_base + 3] = (_sd, lambda a, b: a - b)
    _INT_BIN[_base + 4] = (_sd, _ss)
    _INT_BIN[_base + 5] = (_ud, _su)
_INT_BIN[0x95] = (_V_I16, lambda a, b: a * b)
_INT_BIN[0xAE] = (_V_I32, lambda a, b: a + b)
_INT_BIN[0xB1] = (_V_I32, lambda a, b: a - b)
_INT_BIN[0xB5] = (_V_I32, lambda a, b: a * b)
_INT_BIN[0xCE] = (_V_I64, lambda a, b: a + b)
_INT_BIN[0xD1] = (_V_I64, lambda a, b: a - b)
_INT_BIN[0xD5] = (_V_I64, lambda a, b: a * b)
for _op, _dt in ((0x76, _V_I8), (0x77, _V_U8), (0x96, _V_I16), (0x97, _V_U16), (0xB6, _V_I32), (0xB7, _V_U32)):
    _INT_BIN[_op] = (_dt, np.minimum)
for _op, _dt in ((0x78, _V_I8), (0x79, _V_U8), (0x98, _V_I16), (0x99, _V_U16), (0xB8, _V_I32), (0xB9, _V_U32)):
    _INT_BIN[_op] = (_dt, np.maximum)

_INT_SHIFT = {0x6B: (_V_U8, "l"), 0x6C: (_V_I8, "r"), 0x6D: (_V_U8, "r"), 0x8B: (_V_U16, "l"), 0x8C: (_V_I16, "r"),
              0x8D: (_V_U16, "r"), 0xAB: (_V_U32, "l"), 0xAC: (_V_I32, "r"), 0xAD: (_V_U32, "r"),
              0xCB: (np.dtype("<u8"), "l"), 0xCC: (_V_I64, "r"), 0xCD: (np.dtype("<u8"), "r")}
_INT_EXTEND = {0x87: (_V_I8, _V_I16, 0), 0x88: (_V_I8, _V_I16, 1), 0x89: (_V_U8, _V_U16, 0), 0x8A: (_V_U8, _V_U16, 1),
               0xA7: (_V_I16, _V_I32, 0), 0xA8: (_V_I16, _V_I32, 1), 0xA9: (_V_U16, _V_U32, 0), 0xAA: (_V_U16, _V_U32, 1),
               0xC7: (_V_I32, _V_I64, 0), 0xC8: (_V_I32, _V_I64, 1), 0xC9: (_V_U32, np.dtype("<u8"), 0),
               0xCA: (_V_U32, np.dtype("<u8"), 1)}
_INT_NARROW = {0x65: (_V_I16, _V_I8), 0x66: (_V_I16, _V_U8), 0x85: (_V_I32, _V_I16), 0x86: (_V_I32, _V_U16)}
_INT_CMP = {}
for _base, _sd, _ud in ((0x23, _V_I8, _V_U8), (0x2D, _V_I16, _V_U16), (0x37, _V_I32, _V_U32)):
    _INT_CMP[_base] = (_sd, np.equal)
    _INT_CMP[_base + 1] = (_sd, np.not_equal)
    _INT_CMP[_base + 2] = (_sd, np.less)
    _INT_CMP[_base + 3] = (_ud, np.less)
    _INT_CMP[_base + 4] = (_sd, np.greater)
    _INT_CMP[_base + 5] = (_ud, np.greater)
    _INT_CMP[_base + 6] = (_sd, np.less_equal)
    _INT_CMP[_base + 7] = (_ud, np.less_equal)
    _INT_CMP[_base + 8] = (_sd, np.greater_equal)
    _INT_CMP[_base + 9] = (_ud, np.greater_equal)

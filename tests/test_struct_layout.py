"""The structs that cross the C ABI by value or by pointer: the ``ctypes`` mirrors must have the fields of the header's
``typedef struct`` blocks, in the same order, at the same offsets (natural alignment, as a C compiler lays them out).
Needs no GPU and does not load the library: it parses ``include/b200exl3.h``."""
import ctypes
import re
from pathlib import Path

import pytest

from mlxl3_b200.linear import Prologue
from mlxl3_b200.stack import _StackOp

HEADER = (Path(__file__).resolve().parent.parent / "include" / "b200exl3.h").read_text()

SIZES = {"int": 4, "float": 4, "int32_t": 4, "uint32_t": 4, "int64_t": 8, "size_t": 8}


def c_fields(struct_name: str):
    """[(name, size, alignment)] of ``typedef struct { ... } struct_name;`` (scalars, pointers, arrays of pointers)."""
    end = re.search(r"\}\s*" + re.escape(struct_name) + r"\s*;", HEADER)
    assert end, f"{struct_name} not found in the header"
    start = HEADER.rfind("typedef struct {", 0, end.start())
    assert start >= 0
    body = re.sub(r"/\*.*?\*/", "", HEADER[start + len("typedef struct {"):end.start()], flags=re.S)
    fields = []
    for decl in filter(None, (d.strip() for d in body.split(";"))):
        m = re.fullmatch(r"(?:const\s+)?([A-Za-z_0-9]+)\s*(\*?)\s*(?:const\s+)?([A-Za-z_0-9]+)(?:\[(\d+)\])?", decl)
        assert m, f"cannot parse field declaration {decl!r} of {struct_name}"
        ctype, star, name, count = m.groups()
        size = 8 if star else SIZES[ctype]
        fields.append((name, size * int(count or 1), size))
    return fields


def c_layout(struct_name: str):
    offset, widest, out = 0, 1, []
    for name, size, align in c_fields(struct_name):
        offset = (offset + align - 1) // align * align
        out.append((name, offset, size))
        offset += size
        widest = max(widest, align)
    return out, (offset + widest - 1) // widest * widest


@pytest.mark.parametrize("mirror,struct_name", [(Prologue, "b200exl3_prologue"), (_StackOp, "b200exl3_stack_op")])
def test_ctypes_mirror_matches_the_header(mirror, struct_name):
    layout, total = c_layout(struct_name)
    mine = [(name, getattr(mirror, name).offset, getattr(mirror, name).size) for name, _ in mirror._fields_]
    assert [f[0] for f in mine] == [f[0] for f in layout], "field names or order differ from the header"
    assert mine == layout
    assert ctypes.sizeof(mirror) == total

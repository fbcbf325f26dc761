"""`generate.proto` without protoc.

A small proto3 parser turns `proto/generate.proto` into a `FileDescriptorProto`; protobuf's runtime then builds
the message classes (`pb.Request`, `pb.Batch`, ...), and the same parse tree feeds :mod:`protogen`, which
emits the C++ codec used by the router.  The reference generates `lorax_server/pb/*_pb2.py` with
`grpcio-tools` at build time (`server/Makefile:11-18`); neither protoc nor grpcio-tools exists here.

Supported subset (all that the contract uses): proto3 messages, enums, scalar / message / enum fields,
`repeated`, `optional`, `oneof`, one `service` with unary rpcs, `//` comments.
"""

from __future__ import annotations

import re
from dataclasses import dataclass, field
from pathlib import Path
from types import SimpleNamespace
from typing import Dict, List, Optional

PROTO_PATH = Path(__file__).resolve().parents[2] / "proto" / "generate.proto"
if not PROTO_PATH.exists():       # installed layout: the proto travels inside the package
    PROTO_PATH = Path(__file__).resolve().parent / "generate.proto"

SCALARS = {
    "double": 1, "float": 2, "int64": 3, "uint64": 4, "int32": 5, "fixed64": 6, "fixed32": 7, "bool": 8, "string": 9,
    "bytes": 12, "uint32": 13, "sfixed32": 15, "sfixed64": 16, "sint32": 17, "sint64": 18,
}
TYPE_MESSAGE, TYPE_ENUM = 11, 14


@dataclass
class FieldDef:
    name: str
    number: int
    type_name: str
    repeated: bool = False
    optional: bool = False
    oneof: Optional[str] = None


@dataclass
class MessageDef:
    name: str
    fields: List[FieldDef] = field(default_factory=list)
    oneofs: List[str] = field(default_factory=list)


@dataclass
class EnumDef:
    name: str
    values: Dict[str, int] = field(default_factory=dict)


@dataclass
class RpcDef:
    name: str
    request: str
    response: str


@dataclass
class ProtoFile:
    package: str
    messages: List[MessageDef]
    enums: List[EnumDef]
    service: str
    rpcs: List[RpcDef]


_TOKEN = re.compile(r"[A-Za-z_][A-Za-z0-9_.]*|\d+|[{}()=;<>,]|\"[^\"]*\"")


def parse_proto(text: str) -> ProtoFile:
    text = re.sub(r"//[^\n]*", "", text)
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    toks = _TOKEN.findall(text)
    i = 0
    package, service = "", ""
    messages: List[MessageDef] = []
    enums: List[EnumDef] = []
    rpcs: List[RpcDef] = []

    def expect(t):
        nonlocal i
        if toks[i] != t:
            raise SyntaxError(f"expected {t!r}, got {toks[i]!r} at token {i}")
        i += 1

    def parse_field(msg: MessageDef, oneof: Optional[str]):
        nonlocal i
        repeated = optional = False
        if toks[i] == "repeated":
            repeated = True
            i += 1
        elif toks[i] == "optional":
            optional = True
            i += 1
        tname, fname = toks[i], toks[i + 1]
        i += 2
        expect("=")
        num = int(toks[i])
        i += 1
        expect(";")
        msg.fields.append(FieldDef(fname, num, tname, repeated, optional, oneof))

    while i < len(toks):
        t = toks[i]
        if t == "syntax":
            i += 4
        elif t == "package":
            package = toks[i + 1]
            i += 3
        elif t == "message":
            msg = MessageDef(toks[i + 1])
            i += 2
            expect("{")
            while toks[i] != "}":
                if toks[i] == "oneof":
                    oname = toks[i + 1]
                    msg.oneofs.append(oname)
                    i += 2
                    expect("{")
                    while toks[i] != "}":
                        parse_field(msg, oname)
                    i += 1
                else:
                    parse_field(msg, None)
            i += 1
            messages.append(msg)
        elif t == "enum":
            en = EnumDef(toks[i + 1])
            i += 2
            expect("{")
            while toks[i] != "}":
                en.values[toks[i]] = int(toks[i + 2])
                i += 4
            i += 1
            enums.append(en)
        elif t == "service":
            service = toks[i + 1]
            i += 2
            expect("{")
            while toks[i] != "}":
                expect("rpc")
                name = toks[i]
                i += 1
                expect("(")
                req = toks[i]
                i += 1
                expect(")")
                expect("returns")
                expect("(")
                resp = toks[i]
                i += 1
                expect(")")
                if toks[i] == "{":
                    i += 2
                if i < len(toks) and toks[i] == ";":
                    i += 1
                rpcs.append(RpcDef(name, req, resp))
            i += 1
        else:
            raise SyntaxError(f"unexpected token {t!r}")
    return ProtoFile(package, messages, enums, service, rpcs)


def load_proto_file(path: Optional[Path] = None) -> ProtoFile:
    return parse_proto(Path(path or PROTO_PATH).read_text())


def build_descriptor(pf: ProtoFile, filename: str = "generate.proto"):
    from google.protobuf import descriptor_pb2
    fd = descriptor_pb2.FileDescriptorProto()
    fd.name = filename
    fd.package = pf.package
    fd.syntax = "proto3"
    enum_names = {e.name for e in pf.enums}
    msg_names = {m.name for m in pf.messages}
    for e in pf.enums:
        ed = fd.enum_type.add()
        ed.name = e.name
        for k, v in e.values.items():
            ev = ed.value.add()
            ev.name, ev.number = k, v
    for m in pf.messages:
        md = fd.message_type.add()
        md.name = m.name
        oneof_index = {}
        for o in m.oneofs:
            oneof_index[o] = len(md.oneof_decl)
            md.oneof_decl.add().name = o
        for f in m.fields:
            fdp = md.field.add()
            fdp.name, fdp.number = f.name, f.number
            fdp.json_name = re.sub(r"_([a-z])", lambda mo: mo.group(1).upper(), f.name)
            fdp.label = 3 if f.repeated else 1
            if f.type_name in SCALARS:
                fdp.type = SCALARS[f.type_name]
            elif f.type_name in enum_names:
                fdp.type = TYPE_ENUM
                fdp.type_name = f".{pf.package}.{f.type_name}"
            elif f.type_name in msg_names:
                fdp.type = TYPE_MESSAGE
                fdp.type_name = f".{pf.package}.{f.type_name}"
            else:
                raise KeyError(f"unknown type {f.type_name} in {m.name}.{f.name}")
            if f.oneof is not None:
                fdp.oneof_index = oneof_index[f.oneof]
            elif f.optional:
                # proto3 optional = synthetic oneof
                fdp.proto3_optional = True
                fdp.oneof_index = len(md.oneof_decl)
                md.oneof_decl.add().name = "_" + f.name
    sd = fd.service.add()
    sd.name = pf.service
    for r in pf.rpcs:
        md = sd.method.add()
        md.name = r.name
        md.input_type = f".{pf.package}.{r.request}"
        md.output_type = f".{pf.package}.{r.response}"
    return fd


_pb_cache = None


def load_pb():
    """-> namespace with one attribute per message class and enum (values as ints), plus
    `SERVICE` (full service name), `RPCS` (name -> (request class, response class))."""
    global _pb_cache
    if _pb_cache is not None:
        return _pb_cache
    from google.protobuf import descriptor_pool, message_factory
    pf = load_proto_file()
    fd = build_descriptor(pf)
    pool = descriptor_pool.DescriptorPool()
    pool.Add(fd)
    ns = SimpleNamespace()
    for m in pf.messages:
        desc = pool.FindMessageTypeByName(f"{pf.package}.{m.name}")
        setattr(ns, m.name, message_factory.GetMessageClass(desc))
    for e in pf.enums:
        setattr(ns, e.name, SimpleNamespace(**e.values))
        for k, v in e.values.items():
            setattr(ns, k, v)
    ns.SERVICE = f"{pf.package}.{pf.service}"
    ns.RPCS = {r.name: (getattr(ns, r.request), getattr(ns, r.response)) for r in pf.rpcs}
    ns.METHOD_IDS = {r.name: i + 1 for i, r in enumerate(pf.rpcs)}
    ns.proto = pf
    _pb_cache = ns
    return ns

"""Puts the reference's Python shard package where `bench.py --impl reference` looks for it.

    python baseline/install_reference.py <path to a checkout of predibase/lorax>

The reference is a poetry project (`server/pyproject.toml`); without the poetry-core backend its "install" is the
package directory itself plus the protobuf stubs that `server/Makefile:11-18` generates with grpcio-tools.  This script
copies `server/lorax_server` unmodified into `baseline/_ref/` and writes `lorax_server/pb/generate_pb2.py` from the
reference's own `proto/generate.proto` (the serialized file descriptor is built by this repository's proto3 parser;
no protoc is needed).  Nothing else is added: third-party packages the reference imports (peft, the flash-attention
layer-norm and rotary extensions, its punica kernels, ...) are used if the machine has them and reported by
`bench.py --impl reference` if it does not.
"""

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

PB2 = '''# Generated from the reference's proto/generate.proto (same content protoc would emit, built without protoc).
from google.protobuf import descriptor_pool as _descriptor_pool
from google.protobuf import symbol_database as _symbol_database
from google.protobuf.internal import builder as _builder

_sym_db = _symbol_database.Default()
DESCRIPTOR = _descriptor_pool.Default().AddSerializedFile({blob!r})
_globals = globals()
_builder.BuildMessageAndEnumDescriptors(DESCRIPTOR, _globals)
_builder.BuildTopDescriptorsAndMessages(DESCRIPTOR, "generate_pb2", _globals)
'''


def main(ref_root: str) -> int:
    from lorax_b200.server import proto
    src = os.path.join(ref_root, "server", "lorax_server")
    dst = os.path.join(HERE, "_ref", "lorax_server")
    if not os.path.isdir(src):
        print(f"no server/lorax_server under {ref_root}")
        return 1
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    shutil.copytree(src, dst)
    pf = proto.load_proto_file(os.path.join(ref_root, "proto", "generate.proto"))
    fd = proto.build_descriptor(pf, "generate.proto")
    os.makedirs(os.path.join(dst, "pb"), exist_ok=True)
    with open(os.path.join(dst, "pb", "__init__.py"), "w"):
        pass
    with open(os.path.join(dst, "pb", "generate_pb2.py"), "w") as f:
        f.write(PB2.format(blob=fd.SerializeToString()))
    print(f"copied {src} -> {dst}; wrote pb/generate_pb2.py ({len(pf.messages)} messages, {len(pf.rpcs)} rpcs)")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1] if len(sys.argv) > 1 else "."))

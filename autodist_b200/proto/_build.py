"""Descriptor construction without ``protoc``.

``declare_file`` turns a compact Python description of a ``.proto`` file into a
``FileDescriptorProto``, registers it in the default descriptor pool and
returns ``{message name: generated class}``. The reference generates the same
classes with ``protoc`` at install time (``setup.py:8-39``).
"""
from google.protobuf import descriptor_pb2, descriptor_pool, message_factory

_F = descriptor_pb2.FieldDescriptorProto
_SCALARS = {
    "string": _F.TYPE_STRING, "bool": _F.TYPE_BOOL, "int32": _F.TYPE_INT32, "int64": _F.TYPE_INT64,
    "float": _F.TYPE_FLOAT, "double": _F.TYPE_DOUBLE, "bytes": _F.TYPE_BYTES,
}


def _fill_message(msg, spec, package, path):
    """spec: {"fields": [(name, type, number, opts)], "enums": {...}, "messages": {...}, "oneofs": [...]}"""
    full = f"{path}.{msg.name}" if path else f".{package}.{msg.name}"
    for ename, values in spec.get("enums", {}).items():
        e = msg.enum_type.add()
        e.name = ename
        for vname, vnum in values:
            v = e.value.add()
            v.name, v.number = vname, vnum
    for mname, mspec in spec.get("messages", {}).items():
        sub = msg.nested_type.add()
        sub.name = mname
        _fill_message(sub, mspec, package, full)
    oneofs = spec.get("oneofs", [])
    for o in oneofs:
        msg.oneof_decl.add().name = o
    for name, ftype, number, opts in spec["fields"]:
        f = msg.field.add()
        f.name, f.number = name, number
        f.label = _F.LABEL_REPEATED if opts.get("repeated") else _F.LABEL_OPTIONAL
        if "oneof" in opts:
            f.oneof_index = oneofs.index(opts["oneof"])
        if ftype in _SCALARS:
            f.type = _SCALARS[ftype]
        elif ftype.startswith("map<"):
            # map<string,string> is sugar for a repeated nested *Entry message with map_entry=true.
            ktype, vtype = [t.strip() for t in ftype[4:-1].split(",")]
            entry = msg.nested_type.add()
            entry.name = "".join(p.capitalize() for p in name.split("_")) + "Entry"
            entry.options.map_entry = True
            for i, (n, t) in enumerate((("key", ktype), ("value", vtype)), start=1):
                ef = entry.field.add()
                ef.name, ef.number, ef.label, ef.type = n, i, _F.LABEL_OPTIONAL, _SCALARS[t]
            f.label = _F.LABEL_REPEATED
            f.type = _F.TYPE_MESSAGE
            f.type_name = f"{full}.{entry.name}"
        elif opts.get("enum"):
            f.type = _F.TYPE_ENUM
            f.type_name = ftype
        else:
            f.type = _F.TYPE_MESSAGE
            f.type_name = ftype


def declare_file(name, package, messages, dependencies=()):
    pool = descriptor_pool.Default()
    fdp = descriptor_pb2.FileDescriptorProto()
    fdp.name, fdp.package, fdp.syntax = name, package, "proto3"
    fdp.dependency.extend(dependencies)
    for mname, spec in messages.items():
        m = fdp.message_type.add()
        m.name = mname
        _fill_message(m, spec, package, "")
    try:
        fd = pool.Add(fdp)
    except TypeError:
        # A second import under another module path finds the file already registered.
        fd = pool.FindFileByName(name)
    if fd is None:
        fd = pool.FindFileByName(name)
    return {mname: message_factory.GetMessageClass(fd.message_types_by_name[mname]) for mname in messages}

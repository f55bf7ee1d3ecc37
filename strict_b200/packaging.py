"""Model tensors beside the bytecode in a .strictbinary file.

A .strictbinary is a ZIP whose entries `<type full name>.bytecode` hold the bytecode of one type
each (Strict.Bytecode/BinaryExecutable.cs:40-61,144-157; entry extension
Strict.Bytecode/Serialization/BinaryType.cs:64). The reference's loader reads only the entries
with that extension, so a Strict program can ship a model in the same file: tensors travel as
further entries that its loader skips,

    model/config.json                the model configuration (the fields of strictb200_model_config)
    model/<tensor name>.tensor       16-byte header (magic "SB2T", dtype code, rank, reserved),
                                     rank x int64 shape, then the raw little-endian data

stored without compression (E4M3 weights of a trained or random model do not compress, and a
stored entry can be read in one piece). Tensor names are those of strictb200_model_set_tensor.
"""
import json
import struct
import zipfile

import numpy as np

BytecodeEntryExtension = ".bytecode"   # BinaryType.cs:64
Extension = ".strictbinary"            # BinaryExecutable.cs:155
TensorEntryExtension = ".tensor"
_MAGIC = b"SB2T"
_DTYPES = {0: np.dtype(np.uint8), 1: np.dtype(np.float32)}
_CODES = {v: k for k, v in _DTYPES.items()}


class InvalidFile(Exception):
    """BinaryExecutable.InvalidFile."""


def _tensor_bytes(array):
    array = np.ascontiguousarray(array)
    if array.dtype not in _CODES:
        raise ValueError(f"tensor dtype {array.dtype} is not uint8 (E4M3 codes) or float32")
    header = _MAGIC + struct.pack("<IIi", _CODES[array.dtype], array.ndim, 0)
    return header + struct.pack(f"<{array.ndim}q", *array.shape) + array.tobytes()


def _tensor_from(data, name):
    if len(data) < 16 or data[:4] != _MAGIC:
        raise InvalidFile(f"{name}: not a tensor entry")
    code, rank, _ = struct.unpack("<IIi", data[4:16])
    if code not in _DTYPES or rank > 8:
        raise InvalidFile(f"{name}: unknown dtype or rank")
    shape = struct.unpack(f"<{rank}q", data[16:16 + 8 * rank])
    body = data[16 + 8 * rank:]
    dt = _DTYPES[code]
    if len(body) != int(np.prod(shape, dtype=np.int64)) * dt.itemsize:
        raise InvalidFile(f"{name}: data size does not match its shape")
    return np.frombuffer(body, dtype=dt).reshape(shape)


def add_model(path, config, tensors):
    """Adds (or replaces) the model entries of the .strictbinary at `path`, keeping every other
    entry — the bytecode — byte for byte. Creates the file if it does not exist."""
    kept = []
    try:
        with zipfile.ZipFile(path) as z:
            for info in z.infolist():
                if not info.filename.startswith("model/"):
                    kept.append((info, z.read(info.filename)))
    except FileNotFoundError:
        pass
    except zipfile.BadZipFile as e:
        raise InvalidFile(str(e))
    with zipfile.ZipFile(path, "w") as z:
        for info, data in kept:
            z.writestr(info, data, compress_type=info.compress_type)
        z.writestr("model/config.json", json.dumps(config, sort_keys=True), compress_type=zipfile.ZIP_DEFLATED)
        for name, array in tensors.items():
            z.writestr("model/" + name + TensorEntryExtension, _tensor_bytes(array), compress_type=zipfile.ZIP_STORED)


def bytecode_entries(path):
    """Type full names whose bytecode the file holds — what the reference's loader reads."""
    with zipfile.ZipFile(path) as z:
        return [n[:-len(BytecodeEntryExtension)] for n in z.namelist() if n.lower().endswith(BytecodeEntryExtension)]


def read_model(path):
    """(config dict, {tensor name: array}) or (None, {}) if the file carries no model."""
    try:
        with zipfile.ZipFile(path) as z:
            names = z.namelist()
            if "model/config.json" not in names:
                return None, {}
            config = json.loads(z.read("model/config.json"))
            tensors = {}
            for n in names:
                if n.startswith("model/") and n.endswith(TensorEntryExtension):
                    tensors[n[len("model/"):-len(TensorEntryExtension)]] = _tensor_from(z.read(n), n)
            return config, tensors
    except zipfile.BadZipFile as e:
        raise InvalidFile(str(e))


def save_model(path, model, names):
    """Reads the named tensors back from a single-rank device model and writes them beside the bytecode."""
    tensors = {}
    for name, (dtype, count) in names.items():
        tensors[name] = model.get_tensor(name, dtype, count)
    add_model(path, model.cfg, tensors)


def load_model(ctx, path):
    """Creates the model the file describes on the context's device and uploads its tensors (each
    rank slices its own shard under tensor parallelism)."""
    from .model import Model
    config, tensors = read_model(path)
    if config is None:
        raise InvalidFile(f"{path} carries no model")
    model = Model(ctx, config)
    for name, array in tensors.items():
        model.set_tensor(name, array.reshape(-1))
    return model

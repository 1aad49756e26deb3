"""The ``.rustllm`` container (counterpart of src/core/serialization.rs), bit-exact:

* 136-byte header: magic ``RUSTLLM\\0``, ``format_version`` (1), model version, parameter count /
  bytes / offset, metadata offset / size, checksum, 64 reserved bytes.  The reference dumps its
  ``#[repr(C)]`` struct (6 uninitialised padding bytes); zeros are written here and anything is
  accepted there on read.
* parameters as little-endian fp32 in 8 MiB chunks with a ``(bytes_done, total)`` progress
  callback;
* metadata as length-prefixed little-endian strings;
* checksum ``c = rotl64(c + bits(p), 1)`` per element in order -- sequential by definition, so
  it is computed on the host inside the streaming reader / writer (``csrc/host/io.cpp``).
"""
from __future__ import annotations

import abc
import io
import os
import struct
from dataclasses import dataclass, field
from typing import BinaryIO, Callable, List, Optional, Tuple

import numpy as np

from ..foundation.error import ProcessingError, internal_error, invalid_input
from ..foundation.types import Version
from ..utils import native

MAGIC = b"RUSTLLM\x00"
FORMAT_VERSION = 1
HEADER_SIZE = 136
_HEADER = struct.Struct("<8sIHHH6xQQQQQQ64x")


@dataclass
class ModelHeader:
    magic: bytes = MAGIC
    format_version: int = FORMAT_VERSION
    model_version: Version = field(default_factory=lambda: Version(1, 0, 0))
    param_count: int = 0
    param_bytes: int = 0
    param_offset: int = HEADER_SIZE
    metadata_offset: int = 0
    metadata_size: int = 0
    checksum: int = 0

    @classmethod
    def new(cls, model_version: Version, param_count: int, param_bytes: int) -> "ModelHeader":
        return cls(model_version=model_version, param_count=param_count, param_bytes=param_bytes)

    def validate(self) -> None:
        if self.magic != MAGIC:
            raise invalid_input("Invalid magic bytes")
        if self.format_version != FORMAT_VERSION:
            raise invalid_input(f"Unsupported format version: {self.format_version}")

    def to_bytes(self) -> bytes:
        v = self.model_version
        return _HEADER.pack(self.magic, self.format_version, v.major, v.minor, v.patch,
                            self.param_count, self.param_bytes, self.param_offset,
                            self.metadata_offset, self.metadata_size, self.checksum)

    @classmethod
    def from_bytes(cls, data: bytes) -> "ModelHeader":
        if len(data) < HEADER_SIZE:
            raise invalid_input("Invalid magic bytes")
        (magic, fv, ma, mi, pa, pc, pb, po, mo, ms, ck) = _HEADER.unpack(data[:HEADER_SIZE])
        h = cls(magic, fv, Version(ma, mi, pa), pc, pb, po, mo, ms, ck)
        h.validate()
        return h


class ModelSerializable(abc.ABC):
    @abc.abstractmethod
    def write_to(self, writer: BinaryIO) -> None: ...

    @classmethod
    @abc.abstractmethod
    def read_from(cls, reader: BinaryIO): ...


def _io_error(msg: str):
    return ProcessingError.failed("io", msg)


class ParameterSerializer:
    """8 MiB chunks of little-endian fp32 with a progress callback (serialization.rs:104-194)."""

    def __init__(self) -> None:
        self.buffer_size = 8 * 1024 * 1024

    new = classmethod(lambda cls: cls())

    def write_parameters(self, writer: BinaryIO, params,
                         progress: Optional[Callable[[int, int], None]] = None) -> int:
        arr = np.ascontiguousarray(np.asarray(params, dtype="<f4")).reshape(-1)
        total = arr.size * 4
        written = 0
        step = self.buffer_size // 4
        for s in range(0, arr.size, step):
            chunk = arr[s:s + step].tobytes()
            try:
                writer.write(chunk)
            except OSError as e:
                raise _io_error(f"Failed to write parameters: {e}") from e
            written += len(chunk)
            if progress:
                progress(written, total)
        return written

    def read_parameters(self, reader: BinaryIO, param_count: int,
                        progress: Optional[Callable[[int, int], None]] = None) -> np.ndarray:
        total = param_count * 4
        out = np.empty(param_count, dtype="<f4")
        step = self.buffer_size // 4
        read = 0
        for s in range(0, param_count, step):
            n = min(step, param_count - s)
            data = reader.read(n * 4)
            if len(data) != n * 4:
                raise _io_error("Failed to read parameters: failed to fill whole buffer")
            out[s:s + n] = np.frombuffer(data, dtype="<f4")
            read += len(data)
            if progress:
                progress(read, total)
        return out


@dataclass
class ModelMetadata:
    architecture: str
    training_config: Optional[str] = None
    custom: List[Tuple[str, str]] = field(default_factory=list)

    @classmethod
    def new(cls, architecture: str) -> "ModelMetadata":
        return cls(architecture)

    def with_custom(self, key: str, value: str) -> "ModelMetadata":
        self.custom.append((key, value))
        return self

    def get(self, key: str) -> Optional[str]:
        for k, v in self.custom:
            if k == key:
                return v
        return None

    def to_bytes(self) -> bytes:
        return native.module().rustllm_metadata_to_bytes(self.architecture, self.training_config,
                                                         list(self.custom))

    @classmethod
    def from_bytes(cls, data: bytes) -> "ModelMetadata":
        try:
            arch, tc, custom = native.module().rustllm_metadata_from_bytes(bytes(data))
        except ValueError as e:
            raise invalid_input(str(e)) from None
        return cls(arch, tc, [tuple(kv) for kv in custom])


def calculate_checksum(params) -> int:
    """``for p in params: c = rotl64(c + u64(bits(p)), 1)`` (serialization.rs:375-385)."""
    arr = np.ascontiguousarray(np.asarray(params, dtype=np.float32)).reshape(-1)
    return int(native.module().rustllm_checksum(arr, 0))


def write_rustllm(path: str, params, metadata: ModelMetadata,
                  progress: Optional[Callable[[int, int], None]] = None) -> ModelHeader:
    """Stream ``header | params | metadata`` to ``path`` natively (one pass, checksum folded in)."""
    arr = np.ascontiguousarray(np.asarray(params, dtype=np.float32)).reshape(-1)
    h = native.module().rustllm_write(path, arr, metadata.architecture, metadata.training_config,
                                      list(metadata.custom), progress)
    return ModelHeader(MAGIC, h["format_version"], Version(*h["model_version"]), h["param_count"],
                       h["param_bytes"], h["param_offset"], h["metadata_offset"],
                       h["metadata_size"], h["checksum"])


def read_rustllm(path: str, progress: Optional[Callable[[int, int], None]] = None
                 ) -> Tuple[ModelHeader, np.ndarray, ModelMetadata]:
    try:
        h, arr, (arch, tc, custom) = native.module().rustllm_read(path, progress)
    except ValueError as e:
        raise invalid_input(str(e)) from None
    except RuntimeError as e:
        msg = str(e)
        if "Checksum mismatch" in msg:
            raise internal_error("Checksum mismatch") from None
        raise _io_error(msg) from None
    header = ModelHeader(MAGIC, h["format_version"], Version(*h["model_version"]), h["param_count"],
                         h["param_bytes"], h["param_offset"], h["metadata_offset"],
                         h["metadata_size"], h["checksum"])
    return header, arr, ModelMetadata(arch, tc, [tuple(kv) for kv in custom])


def write_rustllm_stream(writer: BinaryIO, params, metadata: ModelMetadata,
                         progress: Optional[Callable[[int, int], None]] = None) -> ModelHeader:
    """The reference's ``write_to`` sequence on any seekable stream
    (plugins/model-transformer/src/lib.rs:931-1008)."""
    arr = np.ascontiguousarray(np.asarray(params, dtype=np.float32)).reshape(-1)
    header = ModelHeader.new(Version(1, 0, 0), arr.size, arr.size * 4)
    header.checksum = calculate_checksum(arr)
    start = writer.tell()
    writer.write(header.to_bytes())
    ParameterSerializer().write_parameters(writer, arr, progress)
    mbytes = metadata.to_bytes()
    header.metadata_offset = writer.tell() - start
    header.metadata_size = len(mbytes)
    writer.write(mbytes)
    end = writer.tell()
    writer.seek(start)
    writer.write(header.to_bytes())
    writer.seek(end)
    return header


def read_rustllm_stream(reader: BinaryIO, progress: Optional[Callable[[int, int], None]] = None
                        ) -> Tuple[ModelHeader, np.ndarray, ModelMetadata]:
    start = reader.tell()
    header = ModelHeader.from_bytes(reader.read(HEADER_SIZE))
    reader.seek(start + header.param_offset)
    params = ParameterSerializer().read_parameters(reader, header.param_count, progress)
    if calculate_checksum(params) != header.checksum:
        raise internal_error("Checksum mismatch")
    reader.seek(start + header.metadata_offset)
    meta = ModelMetadata.from_bytes(reader.read(header.metadata_size))
    return header, params, meta

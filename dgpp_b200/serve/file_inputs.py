"""File inputs of the chat endpoint: the `/v1/files` store and `file` content parts.

A `file` part names an uploaded file (`{"file": {"file_id": "file-..."}}`) or carries one inline
(`{"file": {"file_data": "data:<mime>;base64,...", "filename": "notes.txt"}}`).  Either way the part is replaced, in
place, by the file's text: UTF-8 text files as they are, PDFs through an external `pdftotext` when the host has one
(otherwise a 400 that says so).  The store keeps uploads under a directory (or a private temporary one), bounded per
file, per request and in total; ids are `file-` + 24 hex digits of the content hash and the upload time.
(reference counterparts: src/serve/file_inputs.hpp / .cpp -- FileInputs, FileInputConfig, the /v1/files routes.)
"""
from __future__ import annotations

import base64
import binascii
import hashlib
import json
import os
import shutil
import subprocess
import tempfile
import threading
import time
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple


class FileInputError(ValueError):
    def __init__(self, message: str, param: str = "file", status: int = 400, code: str = "invalid_file"):
        super().__init__(message)
        self.param, self.status, self.code = param, status, code


@dataclass
class FileInputConfig:
    directory: str = ""                 # empty: a private, ephemeral store for this process
    pdf_command: str = "pdftotext"
    max_file_bytes: int = 50 << 20
    max_request_bytes: int = 50 << 20
    max_text_bytes: int = 128 << 20
    max_storage_bytes: int = 1 << 30
    pdf_timeout_s: float = 120.0


def parse_multipart(body: bytes, content_type: str) -> Dict[str, Tuple[Optional[str], bytes]]:
    """multipart/form-data -> {field name: (filename or None, bytes)}."""
    ct = content_type or ""
    if "multipart/form-data" not in ct or "boundary=" not in ct:
        raise FileInputError("uploads must be multipart/form-data", "file")
    boundary = ct.split("boundary=", 1)[1].split(";")[0].strip().strip('"').encode()
    out: Dict[str, Tuple[Optional[str], bytes]] = {}
    for part in body.split(b"--" + boundary)[1:]:
        if part.startswith(b"--"):
            break
        head, sep, data = part.lstrip(b"\r\n").partition(b"\r\n\r\n")
        if not sep:
            raise FileInputError("malformed multipart section", "file")
        if data.endswith(b"\r\n"):
            data = data[:-2]
        name = filename = None
        for line in head.split(b"\r\n"):
            if line.lower().startswith(b"content-disposition:"):
                for item in line.split(b";")[1:]:
                    k, _, v = item.strip().partition(b"=")
                    v = v.strip().strip(b'"').decode("utf-8", "replace")
                    if k == b"name":
                        name = v
                    elif k == b"filename":
                        filename = v
        if name is None:
            raise FileInputError("multipart section without a field name", "file")
        out[name] = (filename, data)
    return out


class FileInputs:
    def __init__(self, cfg: Optional[FileInputConfig] = None):
        self.cfg = cfg or FileInputConfig()
        self._tmp = None
        if self.cfg.directory:
            os.makedirs(self.cfg.directory, exist_ok=True)
            self.dir = self.cfg.directory
        else:
            self._tmp = tempfile.TemporaryDirectory(prefix="dgpp-files-")
            self.dir = self._tmp.name
        self._lock = threading.Lock()
        self._meta: Dict[str, dict] = {}
        for fn in sorted(os.listdir(self.dir)):              # adopt what an earlier process left
            if fn.endswith(".json"):
                try:
                    m = json.load(open(os.path.join(self.dir, fn)))
                    if os.path.exists(os.path.join(self.dir, m["id"] + ".bin")):
                        self._meta[m["id"]] = m
                except (OSError, ValueError, KeyError):
                    continue

    # ---- store
    def _used(self) -> int:
        return sum(m["bytes"] for m in self._meta.values())

    def upload(self, data: bytes, filename: str, purpose: str = "user_data") -> dict:
        if not data:
            raise FileInputError("the file is empty", "file")
        if len(data) > self.cfg.max_file_bytes:
            raise FileInputError(f"the file exceeds {self.cfg.max_file_bytes} bytes", "file", 413, "file_too_large")
        with self._lock:
            if self._used() + len(data) > self.cfg.max_storage_bytes:
                raise FileInputError("the file store is full", "file", 507, "storage_full")
            now = time.time_ns()
            fid = "file-" + hashlib.blake2b(data + repr(now).encode(), digest_size=12).hexdigest()
            meta = {"id": fid, "object": "file", "bytes": len(data), "created_at": now // 10 ** 9, "created_ns": now,
                    "filename": os.path.basename(filename or "upload"), "purpose": purpose}
            with open(os.path.join(self.dir, fid + ".bin"), "wb") as f:
                f.write(data)
            with open(os.path.join(self.dir, fid + ".json"), "w") as f:
                json.dump(meta, f)
            self._meta[fid] = meta
        return meta

    def list(self) -> List[dict]:
        with self._lock:
            return sorted(self._meta.values(), key=lambda m: (m.get("created_ns", m["created_at"] * 10 ** 9), m["id"]))

    def get(self, fid: str) -> dict:
        with self._lock:
            m = self._meta.get(fid)
        if m is None:
            raise FileInputError(f"no such file '{fid}'", "file_id", 404, "file_not_found")
        return m

    def content(self, fid: str) -> bytes:
        self.get(fid)
        with open(os.path.join(self.dir, fid + ".bin"), "rb") as f:
            return f.read()

    def delete(self, fid: str) -> dict:
        self.get(fid)
        with self._lock:
            self._meta.pop(fid, None)
            for ext in (".bin", ".json"):
                try:
                    os.unlink(os.path.join(self.dir, fid + ext))
                except OSError:
                    pass
        return {"id": fid, "object": "file", "deleted": True}

    # ---- text extraction
    def extract_text(self, data: bytes, filename: str, mime: str = "", param: str = "file") -> str:
        is_pdf = data[:5] == b"%PDF-" or mime == "application/pdf" or (filename or "").lower().endswith(".pdf")
        if is_pdf:
            exe = shutil.which(self.cfg.pdf_command)
            if exe is None:
                raise FileInputError(f"PDF text extraction needs '{self.cfg.pdf_command}', which this host does not have",
                                     param, 400, "pdf_unavailable")
            with tempfile.NamedTemporaryFile(suffix=".pdf", dir=self.dir) as tmp:
                tmp.write(data)
                tmp.flush()
                try:
                    r = subprocess.run([exe, "-layout", "-enc", "UTF-8", tmp.name, "-"], capture_output=True,
                                       timeout=self.cfg.pdf_timeout_s)
                except subprocess.TimeoutExpired:
                    raise FileInputError("PDF text extraction timed out", param, 400, "pdf_timeout") from None
            if r.returncode != 0:
                raise FileInputError("the PDF could not be read", param, 400, "pdf_unreadable")
            text = r.stdout.decode("utf-8", "replace")
        else:
            if b"\x00" in data[:4096]:
                raise FileInputError("binary files other than PDF are not supported", param, 400, "unsupported_file")
            try:
                text = data.decode("utf-8")
            except UnicodeDecodeError:
                raise FileInputError("text files must be UTF-8", param, 400, "invalid_encoding") from None
        if len(text.encode()) > self.cfg.max_text_bytes:
            raise FileInputError("the extracted text is too large", param, 413, "text_too_large")
        return text

    def part_text(self, part: dict, param: str, budget: List[int]) -> str:
        """Text that replaces one `file` content part.  budget[0]: request bytes left (decremented)."""
        f = part.get("file")
        if not isinstance(f, dict):
            raise FileInputError("file parts need a 'file' object", param)
        if f.get("file_id"):
            meta = self.get(str(f["file_id"]))
            data, name, mime = self.content(meta["id"]), meta["filename"], ""
        elif f.get("file_data"):
            url = f["file_data"]
            if not isinstance(url, str) or not url.startswith("data:") or ";base64," not in url:
                raise FileInputError("file_data must be a base64 data: URI", param + ".file.file_data")
            mime = url[5:].split(";")[0].lower()
            try:
                data = base64.b64decode(url.split(",", 1)[1], validate=True)
            except (binascii.Error, ValueError):
                raise FileInputError("file_data is not valid base64", param + ".file.file_data") from None
            name = str(f.get("filename") or "file")
        else:
            raise FileInputError("file parts need a 'file_id' or 'file_data'", param + ".file")
        if len(data) > self.cfg.max_file_bytes or len(data) > budget[0]:
            raise FileInputError("the request's files exceed the size limit", param, 413, "file_too_large")
        budget[0] -= len(data)
        text = self.extract_text(data, name, mime, param)
        return f"\n[file: {os.path.basename(name)}]\n{text}\n[end of file]\n"

"""The /v1/files store and `file` content parts of the chat endpoint (CPU, fake engine)."""
import base64
import http.client
import json

import pytest

from dgpp_b200.runtime import rt
from dgpp_b200.serve.app import Server
from dgpp_b200.serve.file_inputs import FileInputConfig, FileInputError, FileInputs, parse_multipart


def test_store_limits_and_extraction(tmp_path):
    fi = FileInputs(FileInputConfig(directory=str(tmp_path), max_file_bytes=64, max_storage_bytes=100))
    a = fi.upload(b"hello file", "a.txt")
    assert a["id"].startswith("file-") and a["bytes"] == 10 and fi.content(a["id"]) == b"hello file"
    with pytest.raises(FileInputError) as e:
        fi.upload(b"x" * 65, "big.txt")
    assert e.value.status == 413
    fi.upload(b"y" * 60, "b.txt")
    with pytest.raises(FileInputError) as e:
        fi.upload(b"z" * 40, "c.txt")
    assert e.value.status == 507
    # a second store over the same directory adopts the uploads
    again = FileInputs(FileInputConfig(directory=str(tmp_path)))
    assert [m["filename"] for m in again.list()] == ["a.txt", "b.txt"]
    assert again.delete(a["id"])["deleted"] and len(again.list()) == 1
    with pytest.raises(FileInputError) as e:
        again.get(a["id"])
    assert e.value.status == 404
    assert fi.extract_text("grüße".encode(), "t.txt") == "grüße"
    with pytest.raises(FileInputError):
        fi.extract_text(b"\xff\xfe\x00bad", "t.bin")
    with pytest.raises(FileInputError):
        fi.extract_text(b"caf\xe9", "latin1.txt")
    nopdf = FileInputs(FileInputConfig(pdf_command="definitely-not-installed-pdftotext"))
    with pytest.raises(FileInputError) as e:
        nopdf.extract_text(b"%PDF-1.4 ...", "doc.pdf")
    assert e.value.code == "pdf_unavailable"


def test_multipart_parser():
    body = (b"--XyZ\r\nContent-Disposition: form-data; name=\"purpose\"\r\n\r\nuser_data\r\n"
            b"--XyZ\r\nContent-Disposition: form-data; name=\"file\"; filename=\"n.txt\"\r\nContent-Type: text/plain\r\n\r\n"
            b"line1\r\nline2\r\n--XyZ--\r\n")
    f = parse_multipart(body, "multipart/form-data; boundary=XyZ")
    assert f["purpose"] == (None, b"user_data") and f["file"] == ("n.txt", b"line1\r\nline2")
    with pytest.raises(FileInputError):
        parse_multipart(body, "application/json")


def _req(port, method, path, body=None, ctype="application/json"):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=20)
    c.request(method, path, body, {"Content-Type": ctype} if body is not None else {})
    r = c.getresponse()
    data = r.read()
    c.close()
    return r.status, data


def test_files_routes_and_file_parts():
    tok = rt.Tokenizer.byte_level([], [("<|im_start|>", 256, True), ("<|im_end|>", 257, True)], rt.SplitPattern.Qwen2)
    eng = rt.FakeEngine(slots=4, block_tokens=16, blocks=1024, max_context=4096, vocab=256)
    srv = Server(eng, tok, model_name="fake", eos_ids=[257])
    port = srv.start()
    try:
        up = (b"--B\r\nContent-Disposition: form-data; name=\"purpose\"\r\n\r\nuser_data\r\n"
              b"--B\r\nContent-Disposition: form-data; name=\"file\"; filename=\"notes.txt\"\r\n\r\nthe secret is 42\r\n--B--\r\n")
        st, body = _req(port, "POST", "/v1/files", up, "multipart/form-data; boundary=B")
        assert st == 200, body
        fid = json.loads(body)["id"]
        st, body = _req(port, "GET", "/v1/files")
        assert st == 200 and [m["id"] for m in json.loads(body)["data"]] == [fid]
        assert _req(port, "GET", f"/v1/files/{fid}/content") == (200, b"the secret is 42")
        assert json.loads(_req(port, "GET", f"/v1/files/{fid}")[1])["filename"] == "notes.txt"

        def chat(parts):
            return _req(port, "POST", "/v1/chat/completions", json.dumps(
                {"model": "fake", "max_tokens": 4, "messages": [{"role": "user", "content": parts}]}))

        st, plain = chat([{"type": "text", "text": "read: \n[file: notes.txt]\nthe secret is 42\n[end of file]\n"}])
        st2, by_id = chat([{"type": "text", "text": "read: "}, {"type": "file", "file": {"file_id": fid}}])
        inline = "data:text/plain;base64," + base64.b64encode(b"the secret is 42").decode()
        st3, by_data = chat([{"type": "text", "text": "read: "},
                             {"type": "file", "file": {"file_data": inline, "filename": "notes.txt"}}])
        assert st == st2 == st3 == 200
        # the file's text takes the part's place: same prompt, same (deterministic) answer
        pj, ij, dj = json.loads(plain), json.loads(by_id), json.loads(by_data)
        assert pj["usage"]["prompt_tokens"] == ij["usage"]["prompt_tokens"] == dj["usage"]["prompt_tokens"]
        assert pj["choices"][0]["message"]["content"] == ij["choices"][0]["message"]["content"]
        st, err = chat([{"type": "file", "file": {"file_id": "file-nope"}}])
        assert st == 404 and json.loads(err)["error"]["param"] == "file_id"
        st, err = chat([{"type": "file", "file": {"file_data": "data:text/plain;base64,@@"}}])
        assert st == 400 and json.loads(err)["error"]["param"].endswith(".file.file_data")
        assert json.loads(_req(port, "DELETE", f"/v1/files/{fid}")[1])["deleted"] is True
        assert _req(port, "GET", f"/v1/files/{fid}")[0] == 404
    finally:
        srv.stop()

"""OpenAI-compatible server: native HTTP/SSE front end + native scheduler around a scheduler engine.

    python -m dgpp_b200.serve.app --model tiny --port 8000          (random-init model, byte-level tokenizer)

Threads: the C++ epoll thread owns the sockets; ONE service thread (this module) drains parsed requests,
renders + tokenises them, submits them to the scheduler, runs one scheduler tick per loop turn and turns token
events into SSE chunks / final JSON.  Routes: POST /v1/chat/completions, POST /v1/completions, GET /v1/models,
GET /v1/models/{id}, GET /health, GET /metrics, GET /v1/metrics, GET /metrics/prometheus.
(behavioural spec: apps/dgpp_serve.cpp:1483-1744 serve_openai, src/serve/generation_service.cpp:4300-4439
 engine_pass, docs/openai-compatibility.md:17-135 of the reference.)
"""
from __future__ import annotations

import json
import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import Dict, List, Optional

from ..runtime import rt

DEFAULT_TEMPLATE = ("{% for m in messages %}<|im_start|>{{ m.role }}\n{{ m.content }}<|im_end|>\n{% endfor %}"
                    "{% if add_generation_prompt %}<|im_start|>assistant\n{% endif %}")


@dataclass
class _Live:
    rid: str
    conn: int
    req: dict
    index: int
    group: str
    prompt_tokens: int
    created: int
    decoder: object
    scanner: object
    text: bytearray = field(default_factory=bytearray)
    tokens: int = 0
    cached: int = 0
    first_chunk: bool = True
    finish: str = ""
    tool_parser: object = None
    tool_calls: list = field(default_factory=list)
    slot: int = -1
    logprobs: list = field(default_factory=list)
    t_submit: float = 0.0
    t_first: float = 0.0


TOOL_FORMATS = {"json": rt.ToolFormat.JsonTags, "arg-tags": rt.ToolFormat.ArgTags, "dsml": rt.ToolFormat.Dsml,
                "dsml-spaced": rt.ToolFormat.Dsml, "ns-xml": rt.ToolFormat.NsXml}


class Metrics:
    def __init__(self):
        self.c: Dict[str, float] = {"requests_total": 0, "requests_failed": 0, "prompt_tokens_total": 0,
                                    "completion_tokens_total": 0, "cached_tokens_total": 0, "cancelled_total": 0}
        self.ttft: List[float] = []
        self.buckets = [0.01, 0.025, 0.05, 0.1, 0.25, 0.5, 1, 2.5, 5, 10]

    def prometheus(self, sched_meters: dict, prefix: str = "dgpp_b200") -> str:
        out = []
        for k, v in self.c.items():
            out += [f"# TYPE {prefix}_{k} counter", f"{prefix}_{k} {v:g}"]
        for k, v in sched_meters.items():
            out += [f"# TYPE {prefix}_sched_{k} gauge", f"{prefix}_sched_{k} {v:g}"]
        out.append(f"# TYPE {prefix}_time_to_first_token_seconds histogram")
        for b in self.buckets:
            out.append(f'{prefix}_time_to_first_token_seconds_bucket{{le="{b}"}} {sum(1 for t in self.ttft if t <= b)}')
        out.append(f'{prefix}_time_to_first_token_seconds_bucket{{le="+Inf"}} {len(self.ttft)}')
        out.append(f"{prefix}_time_to_first_token_seconds_sum {sum(self.ttft):g}")
        out.append(f"{prefix}_time_to_first_token_seconds_count {len(self.ttft)}")
        return "\n".join(out) + "\n"


class Server:
    def __init__(self, engine, tokenizer, template_src: str = DEFAULT_TEMPLATE, model_name: str = "dgpp-b200",
                 host: str = "127.0.0.1", port: int = 0, eos_ids: Optional[List[int]] = None,
                 default_max_tokens: int = 256, sched_config=None, tool_format=None, constrain_tools: bool = False,
                 world_leader=None, vision=None, files=None):
        self.engine, self.tok = engine, tokenizer
        self.vision = vision                 # serve.vision_frontend.VisionFrontend: image parts of chat messages
        from .file_inputs import FileInputs
        self.files = files or FileInputs()   # the /v1/files store and `file` content parts
        self.template = rt.ChatTemplate(template_src)
        self.model_name = model_name
        self.eos_ids = eos_ids or []
        self.default_max_tokens = default_max_tokens
        # a name of TOOL_FORMATS or an rt.ToolFormat; "dsml-spaced" is the DSML dialect whose marker is followed by a space
        self.dsml_spaced = tool_format == "dsml-spaced"
        if isinstance(tool_format, str):
            tool_format = TOOL_FORMATS[tool_format]
        self.tool_format = tool_format or rt.ToolFormat.JsonTags
        self.constrain_tools = constrain_tools
        self.throughput_log_s = 10.0
        # multi-rank serving: every scheduler input goes through the journal to the follower ranks first
        self.world = world_leader
        self.sched = rt.Scheduler(engine, sched_config or rt.SchedulerConfig())
        self.http = rt.HttpServer(host, port)
        self.live: Dict[str, _Live] = {}
        self.groups: Dict[str, dict] = {}
        self.metrics = Metrics()
        self.started = int(time.time())
        self._stop = threading.Event()
        self.failed_event = threading.Event()        # set by _fail_engine; the process entry point turns it into exit 2
        self._thread: Optional[threading.Thread] = None
        self.failed: Optional[str] = None
        self._tok_bytes = None

    # ------------------------------------------------------------------ lifecycle
    def start(self) -> int:
        self.http.start()
        self._thread = threading.Thread(target=self._loop, name="dgpp-service", daemon=True)
        self._thread.start()
        return self.http.port()

    def stop(self) -> None:
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=30)
        self.http.stop()
        if self.world is not None:
            self.world.shutdown()

    def port(self) -> int:
        return self.http.port()

    # ------------------------------------------------------------------ loop
    def _throughput_line(self, now: float) -> None:
        """One log line per interval while there was traffic: requests, prompt / completion tokens per second,
        live and queued requests, prefix-hit tokens (the 10 s throughput log of the serving process)."""
        c = self.metrics.c
        dt = now - self._tp_t
        dp, dc, dr = (c["prompt_tokens_total"] - self._tp_last[0], c["completion_tokens_total"] - self._tp_last[1],
                      c["requests_total"] - self._tp_last[2])
        if dp or dc or dr or self.live:
            m = self.sched.meters()
            rt.log("info", "serve", f"throughput: {dr} req, prompt {dp / dt:.1f} tok/s, completion {dc / dt:.1f} tok/s, "
                                    f"live {len(self.live)}, queued {self.sched.queued()}, "
                                    f"prefix hit tokens {m['prefix_hit_tokens']}")
        self._tp_last = (c["prompt_tokens_total"], c["completion_tokens_total"], c["requests_total"])
        self._tp_t = now

    def _loop(self) -> None:
        self._tp_t, self._tp_last = time.time(), (0, 0, 0)
        while not self._stop.is_set():
            if time.time() - self._tp_t >= self.throughput_log_s:
                self._throughput_line(time.time())
            busy = not self.sched.idle() and not self.failed
            for req in self.http.poll(0 if busy else 50):
                try:
                    self._route(req)
                except rt.ApiError as e:
                    self.metrics.c["requests_failed"] += 1
                    self.http.respond(req["conn"], e.args[0], "application/json", e.args[1].encode())
                except Exception as e:  # never let one request kill the loop
                    self.metrics.c["requests_failed"] += 1
                    body = rt.error_json(500, f"internal error: {e}", type="server_error")
                    self.http.respond(req["conn"], 500, "application/json", body.encode())
            for conn in self.http.poll_disconnects():
                for lv in list(self.live.values()):
                    if lv.conn == conn:
                        if self.world is not None:
                            self.world.cancel(self.sched, lv.rid)
                        else:
                            self.sched.cancel(lv.rid)
            if not self.sched.idle() and not self.failed:
                try:
                    if self.world is not None:
                        self.world.tick(self.sched)
                    else:
                        self.sched.tick()
                except Exception as e:
                    # the loop keeps serving the sockets: the error events must leave, later requests get a 503
                    self._fail_engine(str(e))
                    continue
                self._drain_events()

    def _fail_engine(self, why: str) -> None:
        """Engine failure: every open request gets an engine_failure error, the server stops accepting work and, when
        it runs as a process (`main`), the leader exits with status 2 (followers see the closed journal and exit 3)."""
        self.failed = why
        self.failed_event.set()
        rt.log("error", "serve", f"engine failure: {why}")
        err = rt.error_json(500, f"engine failure: {why}", type="engine_failure")
        for lv in list(self.live.values()):
            g = self.groups.get(lv.group)
            if g and g["stream"]:
                self.http.stream_send(lv.conn, f"data: {err}\n\n".encode())
                self.http.stream_end(lv.conn)
            else:
                self.http.respond(lv.conn, 500, "application/json", err.encode())
        self.live.clear()
        self.groups.clear()

    # ------------------------------------------------------------------ routing
    def _route(self, req: dict) -> None:
        path, method, conn = req["path"].rstrip("/") or "/", req["method"], req["conn"]
        if self.failed:
            self.http.respond(conn, 503, "application/json",
                              rt.error_json(503, "engine failed: " + self.failed, type="engine_failure").encode())
            return
        if method == "GET" and path == "/health":
            self.http.respond(conn, 200, "application/json", b'{"status":"ok"}')
        elif method == "GET" and path == "/v1/models":
            self.http.respond(conn, 200, "application/json", rt.models_json([self.model_name], self.started).encode())
        elif method == "GET" and path.startswith("/v1/models/"):
            if path[len("/v1/models/"):] == self.model_name:
                body = json.dumps({"id": self.model_name, "object": "model", "created": self.started, "owned_by": "dgpp_b200"})
                self.http.respond(conn, 200, "application/json", body.encode())
            else:
                self.http.respond(conn, 404, "application/json", rt.error_json(404, "model not found", param="model").encode())
        elif method == "GET" and path in ("/metrics", "/v1/metrics"):
            body = json.dumps({"counters": self.metrics.c, "scheduler": self.sched.meters(), "live": len(self.live),
                               "process": rt.process_memory()})
            self.http.respond(conn, 200, "application/json", body.encode())
        elif method == "GET" and path == "/metrics/prometheus":
            self.http.respond(conn, 200, "text/plain; version=0.0.4", self.metrics.prometheus(self.sched.meters()).encode())
        elif path == "/v1/files" or path.startswith("/v1/files/"):
            self._files_route(conn, method, path, req)
        elif method == "POST" and path in ("/v1/chat/completions", "/v1/completions"):
            self._submit(conn, req["body"].decode("utf-8", "replace"), chat=path.endswith("chat/completions"))
        elif path in ("/v1/chat/completions", "/v1/completions", "/health", "/v1/models"):
            self.http.respond(conn, 405, "application/json", rt.error_json(405, "method not allowed").encode())
        else:
            self.http.respond(conn, 404, "application/json", rt.error_json(404, f"unknown route {path}").encode())

    def _files_route(self, conn: int, method: str, path: str, req: dict) -> None:
        """/v1/files: upload (multipart: file, purpose), list, metadata, content, delete."""
        from .file_inputs import FileInputError, parse_multipart
        try:
            if path == "/v1/files" and method == "POST":
                hdrs = {str(k).lower(): v for k, v in dict(req.get("headers") or {}).items()}
                fields = parse_multipart(req["body"], hdrs.get("content-type", ""))
                if "file" not in fields:
                    raise FileInputError("the upload has no 'file' field", "file")
                name, data = fields["file"]
                purpose = fields.get("purpose", (None, b"user_data"))[1].decode("utf-8", "replace")
                out = self.files.upload(data, name or "upload", purpose)
            elif path == "/v1/files" and method == "GET":
                out = {"object": "list", "data": self.files.list()}
            elif method == "GET" and path.endswith("/content"):
                fid = path[len("/v1/files/"):-len("/content")]
                self.http.respond(conn, 200, "application/octet-stream", self.files.content(fid))
                return
            elif method == "GET":
                out = self.files.get(path[len("/v1/files/"):])
            elif method == "DELETE":
                out = self.files.delete(path[len("/v1/files/"):])
            else:
                self.http.respond(conn, 405, "application/json", rt.error_json(405, "method not allowed").encode())
                return
            self.http.respond(conn, 200, "application/json", json.dumps(out).encode())
        except FileInputError as e:
            self.http.respond(conn, e.status, "application/json",
                              rt.error_json(e.status, str(e), param=e.param, code=e.code).encode())

    def _inline_files(self, messages: list) -> None:
        """Replace every `file` content part by the file's text, in place and in order."""
        from .file_inputs import FileInputError
        budget = [self.files.cfg.max_request_bytes]
        for mi, m in enumerate(messages):
            parts = m.get("parts")
            if not parts or not any(p.get("type") == "file" for p in parts):
                continue
            new = []
            for pi, part in enumerate(parts):
                if part.get("type") == "file":
                    try:
                        text = self.files.part_text(part, f"messages[{mi}].content[{pi}]", budget)
                    except FileInputError as e:
                        raise rt.ApiError(e.status, rt.error_json(e.status, str(e), param=e.param, code=e.code)) from None
                    new.append({"type": "text", "text": text})
                else:
                    new.append(part)
            if all(p.get("type") == "text" for p in new):
                m["content"] = "".join(p["text"] for p in new)
                m.pop("parts", None)
            else:
                m["parts"] = new

    def _submit(self, conn: int, body: str, chat: bool) -> None:
        r = rt.parse_chat_request(body) if chat else rt.parse_completion_request(body)
        prepared = None                      # vision: prompt ids + the images' embedding spans
        if chat:
            ctx = {"messages": json.loads(r["messages_json"]), "add_generation_prompt": True}
            tools = json.loads(r["tools_json"])
            if tools:
                ctx["tools"] = tools
            kw = json.loads(r["chat_template_kwargs_json"])
            if kw:
                ctx.update(kw)
            self._inline_files(ctx["messages"])
            if self.vision is not None and self.vision.has_images(ctx["messages"]):
                from .image_inputs import ImageInputError
                if self.world is not None:
                    raise rt.ApiError(400, rt.error_json(400, "images are not served by multi-rank deployments yet",
                                                         param="messages"))
                try:
                    prepared = self.vision.prepare_chat(
                        ctx["messages"], lambda msgs: self.template.render_json(json.dumps({**ctx, "messages": msgs})),
                        self.tok.encode)
                except ImageInputError as e:
                    raise rt.ApiError(400, rt.error_json(400, str(e), param=e.param)) from None
                ids = prepared.ids
            else:
                if any(m.get("parts") for m in ctx["messages"]):
                    raise rt.ApiError(400, rt.error_json(400, "this model does not accept image, audio, video or file "
                                                         "content parts", param="messages"))
                ids = self.tok.encode(self.template.render_json(json.dumps(ctx)))
        elif r["prompt_ids"]:
            ids = list(r["prompt_ids"])
        else:
            ids = self.tok.encode(r["prompt_text"])
        if not ids:
            raise rt.ApiError(400, rt.error_json(400, "the prompt is empty", param="messages" if chat else "prompt"))
        max_tokens = r["max_tokens"] if r["max_tokens"] > 0 else self.default_max_tokens
        if len(ids) + max_tokens > self.engine.max_context():
            raise rt.ApiError(400, rt.error_json(
                400, f"prompt ({len(ids)} tokens) plus max_tokens ({max_tokens}) exceeds the context window "
                     f"({self.engine.max_context()})", param="max_tokens", code="context_length_exceeded"))
        group = ("chatcmpl-" if chat else "cmpl-") + uuid.uuid4().hex[:24]
        created = int(time.time())
        self.groups[group] = {"conn": conn, "chat": chat, "stream": r["stream"], "n": r["n"], "done": 0, "req": r,
                              "choices": [None] * r["n"], "created": created, "prompt_tokens": len(ids)}
        self.metrics.c["requests_total"] += 1
        self.metrics.c["prompt_tokens_total"] += len(ids)
        if r["stream"]:
            self.http.stream_begin(conn)
        params, schema = self._sampling_of(r)
        real_ids = prepared.real_ids if prepared is not None else ids
        if prepared is not None:
            self.groups[group]["image_tokens"] = prepared.image_tokens
        for i in range(r["n"]):
            rid = f"{group}-{i}"
            if prepared is not None:
                self.engine.set_embeds(rid, prepared.spans)
            tool_mode = self._tool_constraint(r) if chat else None
            if (params is not None or schema is not None or tool_mode is not None) and hasattr(self.engine, "configure"):
                if params is not None and r["n"] > 1 and r["seed"] is not None:
                    params = type(params)(**{**params.__dict__, "seed": int(r["seed"]) + i})
                grammar, spec = None, None
                if tool_mode is not None:
                    required, only = tool_mode
                    par = bool(r.get("parallel_tool_calls", True))
                    grammar = rt.ToolGrammar(r["tools_json"], required, par, self._token_table(), self.eos_ids, only)
                    spec = ["tools", r["tools_json"], required, par, only]
                elif schema is not None:
                    grammar = rt.JsonGrammar(schema, self._token_table(), self.eos_ids)
                    spec = ["json", schema]
                if self.world is not None:
                    self.world.configure(rid, None if params is None else dict(params.__dict__), spec, ids)
                self.engine.configure(rid, params, grammar, real_ids)
            self.live[rid] = _Live(rid, conn, r, i, group, len(ids), created, rt.StreamDecoder(self.tok, True),
                                   rt.StopScanner(list(r["stop"])), t_submit=time.time())
            if chat and r["tools_json"] not in ("null", "[]") and json.loads(r["tool_choice_json"]) != "none":
                self.live[rid].tool_parser = rt.ToolParser(self.tool_format, f"call_{uuid.uuid4().hex[:12]}_")
                if self.tool_format == rt.ToolFormat.NsXml:          # value types come from the tools' parameter schemas
                    self.live[rid].tool_parser.set_tools(r["tools_json"])
                if self.dsml_spaced:
                    self.live[rid].tool_parser.set_dsml_spaced(True)
            kw = dict(eos_ids=[] if r["ignore_eos"] else self.eos_ids, ignore_eos=r["ignore_eos"],
                      prefix_cache=r["prefix_cache"], cache_key=r["prompt_cache_key"])
            if self.world is not None:
                self.world.submit(self.sched, rid, ids, max_tokens, **kw)
            else:
                self.sched.submit(rid, ids, max_tokens, **kw)

    def _tool_constraint(self, r: dict):
        """(required, only-this-function) when the request's tool calls are decoded under the tool grammar, else None.
        tool_choice "required" or a named function forces a call; "auto" is constrained only when the server was
        started with constrain_tools (the text stays free until the model opens a call)."""
        if self.tool_format != rt.ToolFormat.JsonTags or r["tools_json"] in ("null", "[]"):
            return None
        choice = json.loads(r["tool_choice_json"])
        if choice == "none":
            return None
        if choice == "required":
            return True, ""
        if isinstance(choice, dict):
            name = (choice.get("function") or {}).get("name") or choice.get("name") or ""
            names = [(t.get("function") or t).get("name") for t in json.loads(r["tools_json"])]
            if name not in names:
                raise rt.ApiError(400, rt.error_json(400, f"tool_choice names an unknown function {name!r}", param="tool_choice"))
            return True, name
        return (False, "") if self.constrain_tools else None

    def _token_table(self):
        """Raw bytes of every vocabulary entry (specials empty): the grammar's view of the tokenizer."""
        if self._tok_bytes is None:
            n = self.tok.vocab_size()
            self._tok_bytes = [b"" if self.tok.is_special(i) else self.tok.token_bytes(i) for i in range(n)]
        return self._tok_bytes

    def _sampling_of(self, r: dict):
        """(SamplingParams or None, schema text or None) of a parsed request; None / None = plain greedy."""
        from ..sampling.device import SamplingParams

        fmt = json.loads(r["response_format_json"])
        schema = None
        if isinstance(fmt, dict) and fmt.get("type") == "json_object":
            schema = ""
        elif isinstance(fmt, dict) and fmt.get("type") == "json_schema":
            js = fmt.get("json_schema") or {}
            schema = json.dumps(js.get("schema", js))
            try:
                rt.json_machine_check(schema, b"")
            except RuntimeError as e:
                raise rt.ApiError(400, rt.error_json(400, str(e), param="response_format"))
        plain = (r["temperature"] <= 0 and r["repetition_penalty"] == 1.0 and not r["presence_penalty"]
                 and not r["frequency_penalty"] and not r["logit_bias"] and not r["logprobs"])
        if plain:
            return None, schema
        seed = r["seed"] if r["seed"] is not None else int(uuid.uuid4().int & 0x7FFFFFFF)
        return SamplingParams(temperature=r["temperature"], top_k=r["top_k"], top_p=r["top_p"], min_p=r["min_p"],
                              repetition_penalty=r["repetition_penalty"], presence_penalty=r["presence_penalty"],
                              frequency_penalty=r["frequency_penalty"], seed=int(seed),
                              top_logprobs=r["top_logprobs"] if r["logprobs"] else 0,
                              logit_bias={int(k): float(v) for k, v in r["logit_bias"].items()}), schema

    # ------------------------------------------------------------------ events -> responses
    def _drain_events(self) -> None:
        for kind, rid, a, b in self.sched.events():
            lv = self.live.get(rid)
            if lv is None:
                continue
            g = self.groups[lv.group]
            if kind == "admit":
                lv.slot = a
                lv.cached = b
                self.metrics.c["cached_tokens_total"] += b
            elif kind == "token":
                if lv.finish:
                    continue
                if lv.tokens == 0:
                    lv.t_first = time.time()
                    self.metrics.ttft.append(lv.t_first - lv.t_submit)
                lv.tokens += 1
                self.metrics.c["completion_tokens_total"] += 1
                self._note_logprob(lv, g, a)
                piece = lv.scanner.feed(lv.decoder.push(a))
                self._emit(lv, g, piece)
                if lv.scanner.stopped():
                    lv.finish = "stop"
                    if self.world is not None:
                        self.world.cancel(self.sched, rid)
                    else:
                        self.sched.cancel(rid)
            elif kind.startswith("retire"):
                why = kind.split(":", 1)[1]
                if why != "shed" and hasattr(self.engine, "forget"):
                    self.engine.forget(rid)          # (a shed request comes back under the same id)
                if not lv.finish:
                    tail = lv.scanner.feed(lv.decoder.flush())
                    tail += lv.scanner.flush()
                    self._emit(lv, g, tail, final=True)
                    lv.finish = {"length": "length", "stop": "stop", "cancelled": "stop", "error": "error"}.get(why, why)
                    if why == "cancelled":
                        self.metrics.c["cancelled_total"] += 1
                self._finish(lv, g)

    def _emit(self, lv: _Live, g: dict, piece: bytes, final: bool = False) -> None:
        """Routes generated text: plain content is streamed / collected; with tools enabled the text first goes
        through the streaming tool-call parser, whose calls become `tool_calls` deltas."""
        if lv.tool_parser is None:
            self._emit_content(lv, g, piece)
            return
        events = lv.tool_parser.feed(piece) if piece else []
        if final:
            events = list(events) + list(lv.tool_parser.finish())
        for ev in events:
            if ev[0] == "content":
                self._emit_content(lv, g, ev[1])
            else:
                _, index, call_id, name, arguments = ev
                call = {"id": call_id, "type": "function", "function": {"name": name, "arguments": arguments}}
                lv.tool_calls.append(call)
                if g["stream"]:
                    delta = json.dumps([{"index": index, **call}])
                    evt = rt.chunk_event(g["chat"], lv.group, self.model_name, lv.created, lv.index, "",
                                         role_delta=lv.first_chunk and g["chat"], tool_calls_json=delta)
                    lv.first_chunk = False
                    self.http.stream_send(lv.conn, evt.encode())

    def _note_logprob(self, lv: _Live, g: dict, token: int) -> None:
        """Collects (token text, logprob, alternatives) of the token just produced when the request asked for it."""
        if not g["req"]["logprobs"] or lv.slot < 0:
            return
        last = getattr(self.engine, "last_logprobs", None)
        rec = last[lv.slot] if last is not None and lv.slot < len(last) else None
        if rec is None:
            return
        text = lambda i: self.tok.token_bytes(int(i)).decode("utf-8", "replace")
        lv.logprobs.append((text(token), float(rec[0]), [(text(i), float(v)) for i, v in rec[1]]))

    def _emit_content(self, lv: _Live, g: dict, piece: bytes) -> None:
        if not piece and not (g["stream"] and lv.first_chunk and g["chat"]):
            return
        lv.text += piece
        if g["stream"]:
            ev = rt.chunk_event(g["chat"], lv.group, self.model_name, lv.created, lv.index,
                                piece.decode("utf-8", "replace"), role_delta=lv.first_chunk and g["chat"])
            lv.first_chunk = False
            self.http.stream_send(lv.conn, ev.encode())

    def _finish(self, lv: _Live, g: dict) -> None:
        if lv.tool_calls and lv.finish == "stop":
            lv.finish = "tool_calls"
        if g["stream"]:
            ev = rt.chunk_event(g["chat"], lv.group, self.model_name, lv.created, lv.index, "", finish_reason=lv.finish)
            self.http.stream_send(lv.conn, ev.encode())
        g["choices"][lv.index] = (lv.index, lv.text.decode("utf-8", "replace"), lv.finish,
                                  json.dumps(lv.tool_calls) if lv.tool_calls else "", list(lv.logprobs),
                                  bool(g["req"]["logprobs"]) and bool(lv.logprobs))
        g["done"] += 1
        g.setdefault("completion_tokens", 0)
        g["completion_tokens"] += lv.tokens
        g["cached"] = max(g.get("cached", 0), lv.cached)
        del self.live[lv.rid]
        if g["done"] == g["n"]:
            if g["stream"]:
                if g["req"]["include_usage"]:
                    self.http.stream_send(lv.conn, rt.usage_event(g["chat"], lv.group, self.model_name, g["created"],
                                                                  g["prompt_tokens"], g["completion_tokens"],
                                                                  g["cached"]).encode())
                self.http.stream_send(lv.conn, rt.done_event().encode())
                self.http.stream_end(lv.conn)
            else:
                body = rt.completion_json(g["chat"], lv.group, self.model_name, g["created"], g["choices"],
                                          g["prompt_tokens"], g["completion_tokens"], g["cached"])
                self.http.respond(lv.conn, 200, "application/json", body.encode())
            del self.groups[lv.group]


def main(argv=None) -> int:
    import argparse

    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--model", default="tiny", choices=["tiny", "fake", "hybrid-tiny", "hybrid", "glm-flash-tiny", "dory-tiny", "flash-next-tiny",
                                                           "minimax-tiny", "mimo-tiny"])
    ap.add_argument("--family-dir", default="",
                    help="a native family checkpoint (dgpp_b200.loaders.family_io.save_family) served through the runner adapter")
    ap.add_argument("--slots", type=int, default=8)
    ap.add_argument("--max-context", type=int, default=4096, help="hybrid models: tokens per request (prompt + output)")
    ap.add_argument("--prefill-chunk", type=int, default=0, help="hybrid models: rows per prefill pass (0: 256 tiny, 2048 full)")
    ap.add_argument("--snapshot-every", type=int, default=0,
                    help="hybrid models: recurrent-state snapshot spacing in tokens (0: 512 tiny, 2048 full)")
    ap.add_argument("--mtp-depth", type=int, default=0,
                    help="hybrid models: draft this many tokens per step with the MTP head and verify them in the same pass")
    ap.add_argument("--layers", type=int, default=48, help="--model hybrid: layer count (fewer than 48 is a smoke run)")
    ap.add_argument("--config", default="", help="deployment JSON (see dgpp_b200.cli resolve); overrides the flags above")
    ap.add_argument("--tool-format", default="json", choices=sorted(TOOL_FORMATS),
                    help="how the model writes tool calls (the streaming parser's format)")
    ap.add_argument("--mixed-pass", action="store_true",
                    help="a reader's prefill chunk rides in the pass of the decode step (engines with a mixed pass)")
    ap.add_argument("--prefill-budget-busy", type=int, default=0,
                    help="prompt tokens per tick while requests are decoding (0: the scheduler's default)")
    ap.add_argument("--vision", action="store_true",
                    help="tiny model only: attach a random-init vision tower so that chat messages accept image_url parts")
    args = ap.parse_args(argv)
    if args.config:
        return serve_deployment(args.config)
    tok = rt.Tokenizer.byte_level([], [("<|im_start|>", 256, True), ("<|im_end|>", 257, True)], rt.SplitPattern.Qwen2)
    sched_config = None
    if args.model == "fake" and not args.family_dir:
        eng = rt.FakeEngine(slots=args.slots, block_tokens=16, blocks=4096, max_context=8192, vocab=256)
    elif args.model in ("hybrid-tiny", "hybrid") and not args.family_dir:
        # Gated DeltaNet + gated attention + MoE family behind the same scheduler / HTTP surface (needs a GPU).
        # "hybrid" is the full shape (48 layers 3:1, hidden 2048, 512 experts top-10 + shared, head_dim 256, NVFP4
        # weights, random-init); "hybrid-tiny" a four-layer smoke model.
        from ..engine.adapters import HybridEngine
        from ..models.hybrid import HybridConfig, HybridModel, HybridRunner
        from ..models.moe import MoEBlock, MoEConfig

        full = args.model == "hybrid"
        chunk = args.prefill_chunk or (2048 if full else 256)
        every = args.snapshot_every or (2048 if full else 512)
        if full:
            hc = HybridConfig(layers=args.layers, hidden=2048, full_every=4, q_heads=16, kv_heads=2, head_dim=256,
                              gdn_k_heads=16, gdn_v_heads=16, gdn_dk=128, gdn_dv=128, vocab=151936, mtp=args.mtp_depth > 0,
                              moe=MoEConfig(hidden=2048, experts=512, top_k=10, moe_ffn=512, shared_ffn=512, router="softmax"))
            MoEBlock.PREFILL_TERMS = 1
            hm = HybridModel.random_init(hc, "cuda", seed=0, std=0.02, fmt="nvfp4")
        else:
            hc = HybridConfig(layers=4, hidden=512, full_every=4, q_heads=4, kv_heads=2, head_dim=128, gdn_k_heads=2,
                              gdn_v_heads=4, gdn_dk=128, gdn_dv=128, ffn=1024, vocab=4096, mtp=args.mtp_depth > 0,
                              moe=MoEConfig(experts=16, top_k=2, moe_ffn=512, shared_ffn=512))
            hm = HybridModel.random_init(hc, "cuda", seed=0, std=0.05)
        eng = HybridEngine(HybridRunner(hm, max_rows=max(chunk, 256), slots=args.slots, max_seq_len=args.max_context,
                                        device="cuda"),
                           snapshot_every=every, max_snapshots=256 if full else 64, prefill_chunk=chunk,
                           mtp_depth=args.mtp_depth)
        sched_config = rt.SchedulerConfig()
        sched_config.prefill_chunk = chunk
        sched_config.prefill_budget_busy = chunk      # a prefix hit's suffix goes through in one or two ticks
        # ids above the byte vocabulary get a printable piece each, so that streamed chunks carry text for every token
        tok = rt.Tokenizer.byte_level([], [("<|im_start|>", 256, True), ("<|im_end|>", 257, True)] +
                                      [(f"<{i}>", i, False) for i in range(258, hc.vocab)], rt.SplitPattern.Qwen2)
    elif args.family_dir or args.model in ("glm-flash-tiny", "dory-tiny", "flash-next-tiny", "minimax-tiny", "mimo-tiny"):
        # the smaller families behind the generic runner adapter (a native family checkpoint, or random-init smoke
        # models; greedy, needs a GPU)
        from ..engine.adapters import RunnerEngine
        from ..models.moe import MoEConfig

        if args.family_dir:
            from ..loaders.family_io import load_family, runner_for
            runner = runner_for(load_family(args.family_dir, "cuda"), 256, args.slots, args.max_context, "cuda")
        elif args.model == "glm-flash-tiny":
            from ..models.glm_flash import GlmFlashConfig, GlmFlashModel, GlmFlashRunner
            fc = GlmFlashConfig(layers=4, hidden=512, vocab=4096, mla_every=2, k_heads=2, v_heads=4, heads=8, q_lora=256,
                                kv_lora=128, nope=64, rope=32, v_dim=64, ffn=1024,
                                moe=MoEConfig(hidden=512, experts=16, top_k=2, moe_ffn=512, shared_ffn=512))
            runner = GlmFlashRunner(GlmFlashModel.random_init(fc, "cuda", seed=0), 256, args.slots, args.max_context, "cuda")
        elif args.model == "dory-tiny":
            from ..models.dory import DoryConfig, DoryModel, DoryRunner
            runner = DoryRunner(DoryModel.random_init(DoryConfig(vocab=4096), "cuda", seed=0), 256, args.slots,
                                args.max_context, "cuda")
        elif args.model == "mimo-tiny":
            from ..models.mimo import MimoConfig, MimoModel, MimoRunner
            mc = MimoConfig(vocab=4096, moe=MoEConfig(hidden=512, experts=16, top_k=2, moe_ffn=512))
            runner = MimoRunner(MimoModel.random_init(mc, "cuda", seed=0), 256, args.slots, args.max_context, "cuda")
        elif args.model == "minimax-tiny":
            from ..models.minimax import MinimaxConfig, MinimaxModel, MinimaxRunner
            mc = MinimaxConfig(vocab=4096, moe_layers=[False, True, True, True],
                               moe=MoEConfig(hidden=512, experts=16, top_k=2, moe_ffn=512, shared_ffn=512, routed_scaling=2.0,
                                             swiglu_limit=7.0, swiglu_alpha=1.702))
            runner = MinimaxRunner(MinimaxModel.random_init(mc, "cuda", seed=0), 256, args.slots, args.max_context, "cuda")
        else:
            from ..models.flash_next import FlashNextConfig, FlashNextModel, FlashNextRunner
            fc = FlashNextConfig(vocab=4096, moe=MoEConfig(hidden=512, experts=16, top_k=2, moe_ffn=512, shared_ffn=512))
            runner = FlashNextRunner(FlashNextModel.random_init(fc, "cuda", seed=0), 256, args.slots, args.max_context, "cuda")
        eng = RunnerEngine(runner, max_context=args.max_context - 128, prefill_chunk=256)
        sched_config = rt.SchedulerConfig()
        sched_config.prefix_cache = False          # the adapter never resumes from cached blocks
        sched_config.prefill_chunk = 256
    else:
        import torch

        from ..engine.adapters import KernelEngine, ReferenceEngine
        from ..engine.llm_engine import LLMEngine
        from ..models.dense import DenseConfig, DenseModel

        if torch.cuda.is_available():
            cfg = DenseConfig.tiny(vocab=4096)
            model = DenseModel.random_init(cfg, device="cuda", seed=0, std=0.05)
            eng = KernelEngine(LLMEngine(model, max_batch=args.slots, max_seq_len=4096, prefill_chunk=512))
        else:
            cfg = DenseConfig.tiny(vocab=4096, weight_fmt="bf16")
            eng = ReferenceEngine(DenseModel.random_init(cfg, device="cpu", seed=0, std=0.05), slots=args.slots)
    vision = None
    if args.vision and args.model == "tiny":
        vision = tiny_vision_frontend(cfg, "cuda" if torch.cuda.is_available() else "cpu")
    if args.mixed_pass or args.prefill_budget_busy:
        sched_config = sched_config or rt.SchedulerConfig()
        sched_config.mixed_pass = bool(args.mixed_pass)
        if args.prefill_budget_busy:
            sched_config.prefill_budget_busy = args.prefill_budget_busy
    srv = Server(eng, tok, model_name=f"dgpp-b200-{args.model}", host=args.host, port=args.port, eos_ids=[257],
                 vision=vision, sched_config=sched_config, tool_format=args.tool_format)
    print(f"listening on http://{args.host}:{srv.start()}", flush=True)
    try:
        while True:
            time.sleep(3600)
    except KeyboardInterrupt:
        srv.stop()
    return 0


def tiny_vision_frontend(cfg, device: str, seed: int = 0):
    """A random-init vision tower sized for a text config (smoke deployments and tests): 14-pixel patches, 2 x 2 merge,
    image delimiters / pad on ids 1, 2, 3 of the text vocabulary."""
    from ..models.vision import VisionConfig, VisionTower
    from .image_inputs import ImagePreprocess
    from .vision_frontend import VisionFrontend, VisionSpec

    vc = VisionConfig(hidden=256, heads=4, layers=2, mlp=512, out_hidden=cfg.hidden)
    tower = VisionTower.random_init(vc, device=device, seed=seed)
    spec = VisionSpec(start_id=1, pad_id=2, end_id=3, preprocess=ImagePreprocess(grid=vc.grid, min_tokens=4, max_tokens=256))
    return VisionFrontend(tower, spec, cfg.vocab)


def serve_deployment(config_path: str) -> int:
    """Serve what a deployment JSON names: weights through the native loader (or this rank's resident image),
    tokenizer.json and the chat template of the checkpoint directory, engine sized by the config.  `model` may also be
    "fake" / "tiny" (no checkpoint: the launcher's smoke deployments).

    tensor_parallel > 1: start one process per GPU (``python -m torch.distributed.run --nproc-per-node W -m
    dgpp_b200.serve.app --config <json>``).  Rank 0 runs the HTTP front end and journals every scheduler input to the
    other ranks (journal port = port + 1 unless DGPP_JOURNAL_PORT is set), which replay it into their own scheduler and
    engine shard; collectives go through the peer-memory reducer.  A follower exits with status 3 when the leader
    goes away."""
    import os

    text = open(config_path).read()
    cfg_json, digest = rt.parse_cluster_config(text)
    cfg = json.loads(cfg_json)
    rt.set_log_level(cfg["log_level"])
    world = int(cfg["tensor_parallel"])
    rank = int(os.environ.get("RANK", "0")) if world > 1 else 0
    rt.log("info", "serve", f"rank {rank}/{world} config: {cfg_json} digest={digest:016x}")
    eos = [257]
    template = DEFAULT_TEMPLATE
    if cfg["model"] == "fake" or (cfg["model"] == "tiny" and world == 1):
        return main(["--model", cfg["model"], "--host", cfg["host"], "--port", str(cfg["port"]),
                     "--slots", str(cfg["max_concurrency"])])
    import torch

    from ..engine.adapters import KernelEngine
    from ..engine.llm_engine import LLMEngine
    from ..loaders import resident_image
    from ..loaders.checkpoint import dense_config_from_hf, load_dense, open_checkpoint
    from ..models.dense import DenseConfig, DenseModel

    reducer = None
    dev = "cuda"
    if world > 1:
        import torch.distributed as dist

        from ..parallel.peer import PeerReducer
        if int(os.environ.get("WORLD_SIZE", "1")) != world:
            raise SystemExit(f"tensor_parallel {world} wants {world} ranks (torchrun --nproc-per-node {world})")
        local = int(os.environ.get("LOCAL_RANK", rank))
        torch.cuda.set_device(local)
        dev = f"cuda:{local}"
        dist.init_process_group("nccl", device_id=torch.device(dev))
    if cfg["model"] == "tiny":
        dcfg = DenseConfig.tiny(hidden=512, q_heads=8, kv_heads=8, head_dim=128, ffn=2048, vocab=4096, layers=2)
        model = DenseModel.random_init(dcfg, device=dev, seed=0, std=0.05, tp_rank=rank, tp_size=world)
        tok = rt.Tokenizer.byte_level([], [("<|im_start|>", 256, True), ("<|im_end|>", 257, True)], rt.SplitPattern.Qwen2)
        name = "dgpp-b200-tiny"
    else:
        ck = open_checkpoint(cfg["model"])
        dcfg = dense_config_from_hf(ck.config)
        cache_dir = os.environ.get("DGPP_RESIDENT_CACHE_DIR", "")
        build = lambda: load_dense(cfg["model"], device=dev, tp_rank=rank, tp_size=world)
        if cache_dir:
            model, hit = resident_image.load_or_build(build, cache_dir, f"{ck.dir}", dcfg, device=dev, tp_rank=rank,
                                                      tp_size=world)
            rt.log("info", "serve", f"weights from {'the resident image' if hit else 'the checkpoint (image written)'}")
        else:
            model = build()
        tok = rt.Tokenizer.from_file(os.path.join(ck.dir, "tokenizer.json"))
        tc_path = os.path.join(ck.dir, "tokenizer_config.json")
        if os.path.exists(tc_path):
            tc = json.load(open(tc_path))
            template = tc.get("chat_template") or template
            e = tc.get("eos_token")
            e = e.get("content") if isinstance(e, dict) else e
            if e and tok.token_to_id(e) >= 0:
                eos = [tok.token_to_id(e)]
        gen = ck.config.get("eos_token_id")
        if gen is not None:
            eos = sorted(set(eos + (list(gen) if isinstance(gen, list) else [gen])))
        name = os.path.basename(os.path.normpath(ck.dir))
    if world > 1:
        reducer = PeerReducer(dcfg.hidden, cfg["prefill_chunk"], torch.device(dev))
    from ..engine.options import EngineOptions
    eng = KernelEngine(LLMEngine(model, max_batch=cfg["max_concurrency"], max_seq_len=cfg["max_context"],
                                 prefill_chunk=cfg["prefill_chunk"], reducer=reducer, fuse_ar=cfg["fuse_all_reduce"],
                                 options=EngineOptions.from_config(cfg)))
    sc = rt.SchedulerConfig()
    sc.prefill_chunk = int(cfg["prefill_chunk"])
    sc.prefill_group_max = int(cfg["prefill_group_max"])
    sc.mixed_pass = bool(cfg.get("mixed_pass", False))
    leader = None
    if world > 1:
        from .world import WorldLeader, run_follower
        jport = int(os.environ.get("DGPP_JOURNAL_PORT", cfg["port"] + 1))
        if rank != 0:
            table = [b"" if tok.is_special(i) else tok.token_bytes(i) for i in range(tok.vocab_size())]

            def configure(rid, params, grammar_spec, ids):
                from ..sampling.device import SamplingParams
                g = None
                if grammar_spec and grammar_spec[0] == "json":
                    g = rt.JsonGrammar(grammar_spec[1], table, eos)
                elif grammar_spec and grammar_spec[0] == "tools":
                    g = rt.ToolGrammar(grammar_spec[1], grammar_spec[2], grammar_spec[3], table, eos, grammar_spec[4])
                if params is not None:
                    params = SamplingParams(**{**params, "logit_bias": {int(k): v for k, v in params.get("logit_bias", {}).items()}})
                eng.configure(rid, params, g, ids)

            return run_follower(eng, os.environ.get("MASTER_ADDR", "127.0.0.1"), jport, config_digest=digest,
                                on_configure=configure, sched_config=sc)
        leader = WorldLeader(world, jport, config_digest=digest)
        leader.wait_for_followers()
    srv = Server(eng, tok, template_src=template, model_name=name, host=cfg["host"], port=cfg["port"], eos_ids=eos,
                 world_leader=leader, sched_config=sc)
    print(f"listening on http://{cfg['host']}:{srv.start()}", flush=True)
    try:
        while not srv.failed_event.wait(1.0):
            pass
        time.sleep(0.5)            # let the error responses leave the sockets
        srv.stop()
        return 2
    except KeyboardInterrupt:
        srv.stop()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

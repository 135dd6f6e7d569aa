"""HTTP front end (crates/inference-server/src/main.rs:23-251): GET /health, /ready, /v1/metadata, /metrics and
POST /v1/infer (one Linear artifact, {"input": [[f32]]} -> {"output": [[f32]]}) plus POST /v1/generate for the
decoder engine ({"prompt": [ids], "max_tokens": n} -> {"tokens": [ids]}).  Standard-library server; the model is never
entered concurrently: /v1/infer goes through a bounded InferencePool, /v1/generate through one EngineLoop thread that
batches the requests of all handlers continuously.

    python -m rustral_b200.serve.http_server --artifact linear.safetensors --in-features 4 --out-features 3 --bias
    python -m rustral_b200.serve.http_server --model llama-8b --device cuda:0 --weights llama.safetensors --bind 0.0.0.0:8080
"""
from __future__ import annotations

import argparse
import json
import signal
import threading
import time
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

import torch

from ..runtime.inference import InferencePool


class ServerState:
    def __init__(self, infer_fn=None, generate_fn=None, metadata=None, workers: int = 1, queue_bound: int = 64,
                 generate_workers: int = 1, engine_loop=None):
        self.metadata = metadata or {}
        self.ready = True
        self.requests_total = 0
        self.errors_total = 0
        self.latency_ns_sum = 0
        self.lock = threading.Lock()
        self.infer_pool = InferencePool(workers, queue_bound, infer_fn) if infer_fn else None
        # with an engine loop the handlers only wait on their own request, so many may be in flight at once
        self.generate_pool = InferencePool(generate_workers, queue_bound, generate_fn) if generate_fn else None
        self.engine_loop = engine_loop

    def record(self, ns: int, ok: bool) -> None:
        with self.lock:
            self.requests_total += 1
            self.latency_ns_sum += ns
            if not ok:
                self.errors_total += 1

    def prometheus(self) -> str:
        with self.lock:
            return ("# TYPE rustral_infer_requests_total counter\n"
                    f"rustral_infer_requests_total {self.requests_total}\n"
                    "# TYPE rustral_infer_errors_total counter\n"
                    f"rustral_infer_errors_total {self.errors_total}\n"
                    "# TYPE rustral_infer_latency_ns_sum counter\n"
                    f"rustral_infer_latency_ns_sum {self.latency_ns_sum}\n")

    def shutdown(self):
        for p in (self.infer_pool, self.generate_pool):
            if p is not None:
                p.shutdown()
        if self.engine_loop is not None:
            self.engine_loop.shutdown()


class BadRequest(Exception):
    pass


def make_handler(state: ServerState):
    class Handler(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"

        def log_message(self, fmt, *args):   # quiet by default
            pass

        def _send(self, code: int, body, ctype="application/json"):
            data = body if isinstance(body, bytes) else (body if isinstance(body, str) else json.dumps(body)).encode()
            self.send_response(code)
            self.send_header("Content-Type", ctype)
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)

        def do_GET(self):
            if self.path == "/health":
                self._send(200, {"status": "ok"})
            elif self.path == "/ready":
                self._send(200 if state.ready else 503, {"ready": state.ready})
            elif self.path == "/v1/metadata":
                self._send(200, state.metadata)
            elif self.path == "/metrics":
                self._send(200, state.prometheus(), "text/plain; version=0.0.4")
            else:
                self._send(404, {"error": "not found"})

        def do_POST(self):
            t0 = time.perf_counter_ns()
            ok = False
            try:
                n = int(self.headers.get("Content-Length", "0"))
                try:
                    body = json.loads(self.rfile.read(n) or b"{}")
                except json.JSONDecodeError as e:
                    raise BadRequest(f"invalid JSON: {e}")
                if self.path == "/v1/infer" and state.infer_pool is not None:
                    out = state.infer_pool.infer(body)
                elif self.path == "/v1/generate" and state.generate_pool is not None:
                    out = state.generate_pool.infer(body)
                else:
                    self._send(404, {"error": "not found"})
                    return
                ok = True
                self._send(200, out)
            except BadRequest as e:
                self._send(400, {"error": str(e)})
            except Exception as e:   # noqa: BLE001 - a handler must always answer
                self._send(500, {"error": f"{type(e).__name__}: {e}"})
            finally:
                state.record(time.perf_counter_ns() - t0, ok)

    return Handler


def linear_infer_fn(linear, in_features: int):
    """Validation of the reference server: non-empty batch, every row of length in_features (main.rs:203-214)."""
    from ..core import ForwardCtx

    def fn(body):
        rows = body.get("input")
        if not isinstance(rows, list) or len(rows) == 0:
            raise BadRequest("input must be a non-empty list of rows")
        for r in rows:
            if not isinstance(r, list) or len(r) != in_features:
                raise BadRequest(f"every row must have {in_features} values")
        dev = linear.weight.tensor.device
        x = torch.tensor(rows, dtype=torch.float32).to(dev, linear.weight.tensor.dtype)
        with torch.no_grad():
            y = linear(x, ForwardCtx.inference())
        return {"output": y.float().cpu().tolist()}

    return fn


class EngineLoop:
    """One thread owns the engine: it takes submissions from the request handlers, steps the engine while there is
    work, and wakes each handler when its request completes.  Requests that arrive while others are generating join
    the running batch at the next iteration (continuous batching across HTTP requests), instead of queueing behind a
    whole generation."""

    def __init__(self, engine, max_pending: int = 256):
        import queue
        self.engine = engine
        self._inbox: "queue.Queue" = queue.Queue(maxsize=max_pending)
        self._waiting: dict = {}                     # request id -> (result box, event) of the handler waiting for it
        self.steps = 0
        self.failed_steps = 0
        self.last_error = None
        self._stop = False
        self._thread = threading.Thread(target=self._run, daemon=True, name="rustral-engine-loop")
        self._thread.start()

    def _admit(self, item) -> None:
        prompt, max_tokens, box, ev = item
        try:
            self._waiting[self.engine.submit(prompt, max_tokens)] = (box, ev)
        except Exception as e:   # noqa: BLE001 - delivered to the waiting handler
            box.append((False, e))
            ev.set()

    def _deliver(self) -> None:
        """Hands finished requests to their handlers and drops their records."""
        eng = self.engine
        eng.scheduler._retire()
        for r in list(eng.scheduler.completed):
            w = self._waiting.pop(r.id, None)
            if w is not None:
                w[0].append((True, list(r.generated)))
                w[1].set()
            eng.release(r.id)

    def _run(self) -> None:
        import queue
        eng = self.engine
        if eng.runner.device.type == "cuda":         # the current device is per thread
            torch.cuda.set_device(eng.runner.device)
        while not self._stop:
            try:                                     # block only when the engine is idle
                item = self._inbox.get(timeout=0.05) if not eng.scheduler.has_work() else self._inbox.get_nowait()
                self._admit(item)
                continue                             # take everything that is waiting before the next step
            except queue.Empty:
                pass
            if eng.scheduler.has_work():
                try:
                    eng.step()
                    self.steps += 1
                except Exception as e:   # noqa: BLE001 - a failed step must not strand the waiting handlers
                    # the requests of the failed step leave the scheduler too: stepping them again would fail again
                    eng.abort_all()
                    self.failed_steps += 1
                    self.last_error = e
                    for box, ev in self._waiting.values():
                        box.append((False, e))
                        ev.set()
                    self._waiting.clear()
                    continue
                self._deliver()

    def generate(self, prompt, max_tokens: int, timeout: float | None = 600.0) -> list:
        box, ev = [], threading.Event()
        self._inbox.put((list(prompt), int(max_tokens), box, ev), timeout=timeout)
        if not ev.wait(timeout):
            raise TimeoutError("generation timed out")
        ok, val = box[0]
        if not ok:
            raise val
        return val

    def shutdown(self) -> None:
        self._stop = True
        self._thread.join(timeout=10)


def engine_generate_fn(engine, loop: "EngineLoop | None" = None):
    """Handler body of /v1/generate.  With `loop` the request joins the shared engine loop; without it the calling
    thread runs the engine to completion (single-request use)."""
    def fn(body):
        prompt = body.get("prompt")
        if not isinstance(prompt, list) or not prompt or not all(isinstance(t, int) for t in prompt):
            raise BadRequest("prompt must be a non-empty list of token ids")
        vocab = engine.runner.cfg.vocab_size
        if any(t < 0 or t >= vocab for t in prompt):
            raise BadRequest("token id out of range")
        max_tokens = int(body.get("max_tokens", 16))
        try:
            if loop is not None:
                return {"tokens": loop.generate(prompt, max_tokens)}
            return {"tokens": engine.generate(prompt, max_tokens)}
        except ValueError as e:
            raise BadRequest(str(e))

    return fn


def serve(state: ServerState, host: str = "127.0.0.1", port: int = 8080, install_signal_handlers: bool = True):
    """Blocks until SIGINT / SIGTERM (graceful: in-flight requests finish)."""
    httpd = ThreadingHTTPServer((host, port), make_handler(state))
    if install_signal_handlers:
        def stop(*_):
            state.ready = False
            threading.Thread(target=httpd.shutdown, daemon=True).start()
        signal.signal(signal.SIGINT, stop)
        signal.signal(signal.SIGTERM, stop)
    try:
        httpd.serve_forever()
    finally:
        httpd.server_close()
        state.shutdown()
    return httpd


def start_background(state: ServerState, host: str = "127.0.0.1", port: int = 0):
    """Starts the server on a thread (tests, notebooks); returns (httpd, thread).  port 0 picks a free port."""
    httpd = ThreadingHTTPServer((host, port), make_handler(state))
    th = threading.Thread(target=httpd.serve_forever, daemon=True)
    th.start()
    return httpd, th


def build_state(a) -> ServerState:
    """The server state for parsed command-line arguments: a Linear artifact behind /v1/infer, or a decoder engine
    (continuous batching over the paged KV cache) behind /v1/generate."""
    from ..core import B200Backend, CpuBackend
    if a.model:
        from ..models.config import preset
        from .engine import ServingEngine
        from .model_runner import ModelRunner
        cfg = preset(a.model, **({"n_layer": a.layers} if a.layers else {}))
        params = None
        if a.device != "cpu" and cfg.arch == "llama":
            from .weights import InferenceWeights           # bf16 inference weights (no optimizer buffers)
            params = InferenceWeights.random_llama(cfg, a.device, 0, 1, a.seed)
        runner = ModelRunner(cfg, params=params, device=a.device, num_blocks=a.blocks, block_size=a.page, seed=a.seed)
        if a.weights:
            from ..io import safetensors_io as st
            tensors, _ = st.load_file(a.weights)            # strict: names and shapes must match the preset
            if hasattr(runner.params, "tensors"):
                runner.params.load_state_dict(tensors, cfg)
            else:
                runner.params.load_state_dict(tensors)
        engine = ServingEngine(runner, max_batch_size=a.max_batch, eos_id=a.eos_id)
        engine.generate([1, 2, 3], 2)                       # warm-up: compiles nothing, but touches every kernel once
        meta = {"model": a.model, "layers": cfg.n_layer, "d_model": cfg.d_model, "vocab_size": cfg.vocab_size,
                "context": cfg.seq_len, "page_size": a.page, "kv_blocks": a.blocks, "device": a.device,
                "weights": a.weights or "random-init"}
        loop = EngineLoop(engine)
        return ServerState(generate_fn=engine_generate_fn(engine, loop), metadata=meta, generate_workers=a.max_batch,
                           engine_loop=loop)
    if not a.artifact or not a.in_features or not a.out_features:
        raise SystemExit("give --model NAME (decoder engine) or --artifact FILE --in-features N --out-features M (Linear)")
    from ..nn.linear import LinearBuilder
    from ..runtime.model_io import load_model_from_path
    backend = CpuBackend() if a.device == "cpu" else B200Backend()
    lin = LinearBuilder(a.in_features, a.out_features).with_bias(a.bias).build(backend)
    load_model_from_path(lin, a.artifact)          # strict: missing / extra keys and shape mismatches are errors
    return ServerState(linear_infer_fn(lin, a.in_features),
                       metadata={"model": "linear", "in_features": a.in_features, "out_features": a.out_features,
                                 "bias": a.bias, "backend": backend.name})


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description="rustral-b200 inference server")
    ap.add_argument("--bind", default="127.0.0.1:8080")
    ap.add_argument("--device", default="cpu")
    g = ap.add_argument_group("Linear artifact (/v1/infer)")
    g.add_argument("--artifact", help="safetensors file of one Linear (keys weight, bias)")
    g.add_argument("--in-features", type=int, default=0)
    g.add_argument("--out-features", type=int, default=0)
    g.add_argument("--bias", action="store_true")
    e = ap.add_argument_group("decoder engine (/v1/generate)")
    e.add_argument("--model", help="model preset, e.g. llama-8b, gpt2-small")
    e.add_argument("--layers", type=int, default=0, help="override the preset's depth")
    e.add_argument("--weights", help="safetensors state dict of the model; random-init when absent")
    e.add_argument("--blocks", type=int, default=4096, help="KV-cache pages")
    e.add_argument("--page", type=int, default=16, help="tokens per KV-cache page")
    e.add_argument("--max-batch", type=int, default=64)
    e.add_argument("--eos-id", type=int, default=None)
    e.add_argument("--seed", type=int, default=0)
    return ap.parse_args(argv)


def main(argv=None):
    a = parse_args(argv)
    state = build_state(a)
    host, port = a.bind.rsplit(":", 1)
    serve(state, host, int(port))


if __name__ == "__main__":
    main()

"""Least-in-flight load balancer in front of several server replicas (one process per GPU).

    # eight single-GPU replicas on ports 8000..8007 and the balancer on 9000
    python -m sensenova_u1_b200.serving.balancer --replicas 8 --model_path CKPT --port 9000
    # or in front of servers that already run
    python -m sensenova_u1_b200.serving.balancer --backends http://127.0.0.1:8000,http://127.0.0.1:8001

Clients (benchmark harnesses, the serving client) see one OpenAI-style endpoint.  Every request goes to the healthy
replica with the fewest requests in flight (ties: the one chosen least recently); a replica that stops answering
``/health`` is skipped until it answers again; streamed answers pass through chunk by chunk.  ``GET /_lb/status``
shows the table.  Role of the reference's evaluation/easi/scripts/lb.py:1-213 and of the data-parallel branch of
evaluation/easi/scripts/serve.sh (replicas + balancer from one command)."""
import argparse
import asyncio
import os
import signal
import subprocess
import sys
import time
from contextlib import asynccontextmanager
from typing import Dict, List, Optional, Sequence

_HOP = {"host", "content-length", "connection", "transfer-encoding", "keep-alive", "upgrade"}


class Backends:
    """In-flight counters and health flags of the replicas."""

    def __init__(self, urls: Sequence[str]):
        self.urls: List[str] = [u.strip().rstrip("/") for u in urls if u.strip()]
        if not self.urls:
            raise ValueError("no backends given")
        self.inflight: Dict[str, int] = {u: 0 for u in self.urls}
        self.healthy: Dict[str, bool] = {u: False for u in self.urls}
        self.served: Dict[str, int] = {u: 0 for u in self.urls}
        self._last: Dict[str, int] = {u: 0 for u in self.urls}
        self._tick = 0

    def pick(self) -> str:
        """Fewest requests in flight among the healthy replicas; with none healthy, among all (the caller then gets
        the replica's own error instead of a made-up one)."""
        cand = [u for u in self.urls if self.healthy[u]] or self.urls
        u = min(cand, key=lambda b: (self.inflight[b], self._last[b]))
        self._tick += 1
        self._last[u] = self._tick
        return u

    def enter(self, u: str) -> None:
        self.inflight[u] += 1
        self.served[u] += 1

    def leave(self, u: str) -> None:
        self.inflight[u] = max(0, self.inflight[u] - 1)

    def mark(self, u: str, ok: bool) -> bool:
        changed = self.healthy[u] != ok
        self.healthy[u] = ok
        return changed

    def status(self) -> dict:
        return {"backends": self.urls, "healthy": dict(self.healthy), "inflight": dict(self.inflight), "served": dict(self.served)}


async def probe(client, url: str, timeout: float = 5.0) -> bool:
    """A replica is up when ``/health`` answers 200 with JSON (a stray listener on the port does not)."""
    try:
        r = await client.get(url + "/health", timeout=timeout)
        return r.status_code == 200 and "json" in r.headers.get("content-type", "").lower()
    except Exception:
        return False


def create_balancer_app(urls: Sequence[str], request_timeout: float = 1800.0, health_interval: float = 10.0,
                        startup_timeout: float = 600.0, client=None):
    """``client``: an ``httpx.AsyncClient`` to use for the replicas (tests pass one with a mock transport)."""
    import httpx
    from fastapi import FastAPI, Request
    from fastapi.responses import JSONResponse, StreamingResponse

    state = Backends(urls)

    async def health_loop(c):
        while True:
            for u in state.urls:
                if state.mark(u, await probe(c, u)):
                    print(f"[lb] {u}: {'up' if state.healthy[u] else 'down'}", flush=True)
            await asyncio.sleep(health_interval)

    @asynccontextmanager
    async def lifespan(app):
        c = client or httpx.AsyncClient(timeout=httpx.Timeout(request_timeout),
                                        limits=httpx.Limits(max_keepalive_connections=128, max_connections=256))
        app.state.client = c
        deadline = time.monotonic() + startup_timeout
        while time.monotonic() < deadline:                      # do not accept work before one replica can take it
            ups = [u for u in state.urls if await probe(c, u)]
            if ups:
                for u in ups:
                    state.mark(u, True)
                break
            await asyncio.sleep(min(2.0, max(0.05, startup_timeout / 10)))
        else:
            print(f"[lb] no replica answered within {startup_timeout:.0f} s; serving anyway", file=sys.stderr, flush=True)
        task = asyncio.create_task(health_loop(c))
        try:
            yield
        finally:
            task.cancel()
            if client is None:
                await c.aclose()

    app = FastAPI(title="sensenova-u1_b200 balancer", lifespan=lifespan)
    app.state.backends = state

    @app.get("/_lb/status")
    async def status():
        return state.status()

    @app.api_route("/{path:path}", methods=["GET", "POST", "PUT", "DELETE", "PATCH", "OPTIONS", "HEAD"])
    async def proxy(path: str, request: Request):
        u = state.pick()
        url = f"{u}/{path}" + (f"?{request.url.query}" if request.url.query else "")
        headers = {k: v for k, v in request.headers.items() if k.lower() not in _HOP}
        body = await request.body()
        c = request.app.state.client
        state.enter(u)
        try:
            up = await c.send(c.build_request(request.method, url, content=body or None, headers=headers), stream=True)
        except Exception as e:
            state.leave(u)
            state.mark(u, False)                                # skipped until the next probe finds it again
            return JSONResponse({"error": f"replica {u} unreachable: {type(e).__name__}: {e}"}, status_code=502)

        async def chunks():
            try:
                if up.is_stream_consumed:                        # a body that arrived whole
                    yield up.content
                else:
                    async for part in up.aiter_raw():
                        yield part
            finally:
                await up.aclose()
                state.leave(u)
        out = {k: v for k, v in up.headers.items() if k.lower() not in _HOP}
        return StreamingResponse(chunks(), status_code=up.status_code, headers=out, media_type=up.headers.get("content-type"))

    return app


def replica_commands(n: int, base_port: int, server_args: Sequence[str], host: str = "127.0.0.1", gpus: Optional[Sequence[int]] = None):
    """(command, environment additions, url) of each replica: one GPU and one port apiece."""
    gpus = list(gpus) if gpus is not None else list(range(n))
    if len(gpus) < n:
        raise ValueError(f"{n} replicas need {n} GPU indexes, got {gpus}")
    out = []
    for i in range(n):
        cmd = [sys.executable, "-m", "sensenova_u1_b200.serving.server", "--host", host, "--port", str(base_port + i), *server_args]
        out.append((cmd, {"CUDA_VISIBLE_DEVICES": str(gpus[i])}, f"http://{host}:{base_port + i}"))
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--backends", default=os.environ.get("BACKENDS", ""), help="comma-separated replica URLs")
    ap.add_argument("--replicas", type=int, default=0, help="start this many single-GPU servers first (ports --replica_port ...)")
    ap.add_argument("--replica_port", type=int, default=8000)
    ap.add_argument("--gpus", default=None, help="GPU indexes of the replicas, e.g. 0,1,2,3 (default 0..replicas-1)")
    ap.add_argument("--host", default=os.environ.get("LB_HOST", "127.0.0.1"))
    ap.add_argument("--port", type=int, default=int(os.environ.get("LB_PORT", 9000)))
    ap.add_argument("--request_timeout", type=float, default=float(os.environ.get("LB_REQUEST_TIMEOUT", 1800)))
    ap.add_argument("--health_interval", type=float, default=float(os.environ.get("LB_HEALTH_INTERVAL", 10)))
    ap.add_argument("--startup_timeout", type=float, default=float(os.environ.get("LB_STARTUP_TIMEOUT", 600)))
    a, server_args = ap.parse_known_args(argv)                 # what is left goes to the replicas (--model_path ...)
    urls = [u for u in a.backends.split(",") if u.strip()]
    children: List[subprocess.Popen] = []
    if a.replicas:
        gpus = [int(g) for g in a.gpus.split(",")] if a.gpus else None
        for cmd, env, url in replica_commands(a.replicas, a.replica_port, server_args, gpus=gpus):
            children.append(subprocess.Popen(cmd, env={**os.environ, **env}))
            urls.append(url)
    elif server_args:
        ap.error(f"unknown arguments {server_args} (server flags need --replicas)")
    import uvicorn
    try:
        uvicorn.run(create_balancer_app(urls, a.request_timeout, a.health_interval, a.startup_timeout), host=a.host,
                    port=a.port, log_level="info", access_log=False)
    finally:
        for p in children:                                      # exactly the processes started above
            if p.poll() is None:
                p.send_signal(signal.SIGTERM)
        for p in children:
            try:
                p.wait(timeout=30)
            except subprocess.TimeoutExpired:
                p.kill()


if __name__ == "__main__":
    main()

"""Pipeline frequency optimizer: plan server and per-rank client.

The server answers "which clocks does pipeline stage p use this step" from a
``freqs_pipeline_*.py`` file (zeus' ``PointSolution3D`` scheduler behind
``uvicorn zeus.optimizer.pipeline_frequency.server.router:app`` in the reference,
``tests/artifact/run_kareus.sh:373-385``).  The client is driven by the training loop's hooks
(``on_step_begin``, ``on_instruction_begin("forward"|"backward")``, ``on_instruction_end``,
``on_step_end``; ``3rdparty/NeMo/.../megatron_base_model.py:702-736``) and asks the asynchronous
:class:`FrequencyController` to apply each instruction's clock.

Two transports: in-process (the plan object is shared) and HTTP (standard library server; one
server on the master node, ``PFO_PORT`` 7787 in the reference's drivers).  If the server cannot be
reached the client falls back to "no plan": the controller is left alone (maximum clock).
"""
from __future__ import annotations

import json
import threading
import urllib.error
import urllib.request
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple

from ..plan.freqs import FreqPlan, parse_freqs_file

DEFAULT_PORT = 7787


class PointSolution:
    """Serves one fixed frequency plan (one list of ``(kind, MHz)`` per pipeline stage)."""

    def __init__(self, plan: FreqPlan):
        self.plan = plan
        self.registered: Dict[int, dict] = {}

    @classmethod
    def from_file(cls, path) -> "PointSolution":
        return cls(parse_freqs_file(path))

    def register(self, rank: int, info: dict) -> None:
        self.registered[rank] = info

    def schedule_for(self, pp_rank: int) -> List[Tuple[str, int]]:
        if not 0 <= pp_rank < len(self.plan):
            raise IndexError(f"plan has {len(self.plan)} stages, asked for stage {pp_rank}")
        return list(self.plan[pp_rank])


class PFOServer:
    """Tiny HTTP front end for a :class:`PointSolution`."""

    def __init__(self, solution: PointSolution, host: str = "127.0.0.1", port: int = DEFAULT_PORT):
        sol = solution

        class Handler(BaseHTTPRequestHandler):
            def log_message(self, *a):  # quiet
                pass

            def _send(self, code, obj):
                body = json.dumps(obj).encode()
                self.send_response(code)
                self.send_header("Content-Type", "application/json")
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)

            def do_POST(self):
                n = int(self.headers.get("Content-Length", "0"))
                data = json.loads(self.rfile.read(n) or b"{}")
                if self.path == "/register":
                    sol.register(int(data.get("rank", -1)), data)
                    self._send(200, {"ok": True})
                else:
                    self._send(404, {"error": "unknown path"})

            def do_GET(self):
                if self.path.startswith("/schedule/"):
                    try:
                        self._send(200, {"schedule": sol.schedule_for(int(self.path.rsplit("/", 1)[1]))})
                    except (IndexError, ValueError) as e:
                        self._send(400, {"error": str(e)})
                elif self.path == "/health":
                    self._send(200, {"ok": True, "stages": len(sol.plan)})
                else:
                    self._send(404, {"error": "unknown path"})

        self.httpd = ThreadingHTTPServer((host, port), Handler)
        self.port = self.httpd.server_address[1]
        self.url = f"http://{host}:{self.port}"
        self._thread = threading.Thread(target=self.httpd.serve_forever, daemon=True)

    def start(self) -> "PFOServer":
        self._thread.start()
        return self

    def stop(self) -> None:
        self.httpd.shutdown()
        self.httpd.server_close()


class PipelineFrequencyOptimizer:
    """Per-rank client.  ``tp_rank``/``tp_degree`` take the CP-folded coordinate."""

    def __init__(self, rank: int, dp_rank: int, pp_rank: int, tp_rank: int, device_id: int, dp_degree: int,
                 pp_degree: int, tp_degree: int, world_size: int, controller, server_url: Optional[str] = None,
                 solution: Optional[PointSolution] = None, job_metadata: Optional[str] = None,
                 timeout_s: float = 2.0):
        self.rank, self.pp_rank = rank, pp_rank
        self.controller = controller
        self.server_url, self.solution, self.timeout_s = server_url, solution, timeout_s
        self.info = dict(rank=rank, dp_rank=dp_rank, pp_rank=pp_rank, tp_rank=tp_rank, device_id=device_id,
                         dp_degree=dp_degree, pp_degree=pp_degree, tp_degree=tp_degree, world_size=world_size,
                         job_metadata=job_metadata)
        self.schedule: Optional[List[Tuple[str, int]]] = None
        self.fallback = False
        self._pos = 0
        self._register()

    # ------------------------------------------------------------------ transport
    def _register(self) -> None:
        if self.solution is not None:
            self.solution.register(self.rank, self.info)
            return
        if self.server_url is None:
            self.fallback = True
            return
        try:
            req = urllib.request.Request(self.server_url + "/register", data=json.dumps(self.info).encode(),
                                         headers={"Content-Type": "application/json"})
            urllib.request.urlopen(req, timeout=self.timeout_s).read()
        except (urllib.error.URLError, OSError):
            self.fallback = True

    def _fetch(self) -> Optional[List[Tuple[str, int]]]:
        if self.solution is not None:
            return self.solution.schedule_for(self.pp_rank)
        if self.server_url is None or self.fallback:
            return None
        try:
            with urllib.request.urlopen(f"{self.server_url}/schedule/{self.pp_rank}", timeout=self.timeout_s) as r:
                return [(k, int(f)) for k, f in json.loads(r.read())["schedule"]]
        except (urllib.error.URLError, OSError, KeyError, ValueError):
            self.fallback = True
            return None

    # ------------------------------------------------------------------ hooks
    def on_step_begin(self) -> None:
        if self.schedule is None and not self.fallback:
            self.schedule = self._fetch()
        self._pos = 0

    def on_instruction_begin(self, name: str) -> None:
        if not self.schedule:
            return
        if self._pos >= len(self.schedule):
            raise RuntimeError("frequency plan has fewer instructions than the step executes")
        kind, mhz = self.schedule[self._pos]
        if kind != name:
            raise RuntimeError(f"frequency plan/loop mismatch at instruction {self._pos}: plan {kind!r}, loop {name!r}")
        self._pos += 1
        self.controller.set_frequency(mhz)

    def on_instruction_end(self, name: str) -> None:
        pass

    def on_step_end(self) -> None:
        if self.schedule and self._pos != len(self.schedule):
            raise RuntimeError(f"step ended after {self._pos} of {len(self.schedule)} planned instructions")

"""Live endpoint check: /health, /v1/models, one JSON completion, one SSE stream ending in [DONE]
(reference: tools/smoke_http.py, tools/smoke_context.py)."""
from __future__ import annotations

import json
import sys

import requests


def run(url: str, api_key: str = "", timeout: float = 120.0) -> int:
    h = {"Authorization": f"Bearer {api_key}"} if api_key else {}
    report = {}
    try:
        r = requests.get(url + "/health", timeout=10)
        report["health"] = r.json() if r.status_code == 200 else r.status_code
        r = requests.get(url + "/v1/models", headers=h, timeout=10)
        report["models"] = [m["id"] for m in r.json()["data"]]
        body = {"model": report["models"][0], "messages": [{"role": "user", "content": "Say hi."}], "max_tokens": 8,
                "temperature": 0}
        r = requests.post(url + "/v1/chat/completions", json=body, headers=h, timeout=timeout)
        r.raise_for_status()
        j = r.json()
        report["completion"] = {"finish": j["choices"][0]["finish_reason"], "tokens": j["usage"]["completion_tokens"],
                                "request_id": r.headers.get("x-request-id")}
        body["stream"] = True
        chunks, done = 0, False
        with requests.post(url + "/v1/chat/completions", json=body, headers=h, timeout=timeout, stream=True) as s:
            s.raise_for_status()
            for line in s.iter_lines():
                if not line.startswith(b"data: "):
                    continue
                if line == b"data: [DONE]":
                    done = True
                    break
                json.loads(line[6:])
                chunks += 1
        report["stream"] = {"chunks": chunks, "done": done}
        ok = done and chunks > 0
    except Exception as e:                                   # noqa: BLE001 - a smoke test reports, it does not raise
        report["error"] = f"{type(e).__name__}: {e}"
        ok = False
    report["ok"] = ok
    print(json.dumps(report))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(run(*sys.argv[1:3]))

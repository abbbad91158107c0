"""Live endpoint check: /health, /v1/models, one JSON completion, one SSE stream ending in [DONE], and
the incremental context transport (a first turn sent in full, a second turn sent as an append to it, a
turn on a base the server never saw -> 409 context_miss) (reference: tools/smoke_http.py,
tools/smoke_context.py)."""
from __future__ import annotations

import json
import sys

import requests


def context_check(url: str, headers: dict, model: str, timeout: float = 120.0) -> dict:
    """Two turns through POST /v1/context/chat/completions: the second sends only what is new."""
    from .context_transport import chain_all
    hh = dict(headers, **{"X-Titanic-Context": "v1"})
    req = {"model": model, "max_tokens": 4, "temperature": 0}
    first = [json.dumps({"role": "user", "content": "Remember the word heron."})]
    env = {"version": 1, "namespace": "smoke", "id": "c1", "base": None, "append": first, "key": chain_all(first), "request": req}
    r1 = requests.post(url + "/v1/context/chat/completions", json=env, headers=hh, timeout=timeout)
    out = {"first": r1.status_code, "ack": r1.headers.get("X-Titanic-Context-Ack"), "stored": r1.headers.get("X-Titanic-Context-Stored")}
    if r1.status_code != 200:
        return dict(out, ok=False)
    key1 = r1.headers.get("X-Titanic-Context-Key")
    reply = r1.json()["choices"][0]["message"]
    more = [json.dumps({"role": "assistant", "content": reply.get("content") or ""}),
            json.dumps({"role": "user", "content": "Which word?"})]
    env2 = {"version": 1, "namespace": "smoke", "id": "c1", "base": {"key": key1, "keep": 1}, "append": more,
            "key": chain_all(more, key1), "request": req}
    r2 = requests.post(url + "/v1/context/chat/completions", json=env2, headers=hh, timeout=timeout)
    out.update(second=r2.status_code, stored_second=r2.headers.get("X-Titanic-Context-Stored"))
    env3 = dict(env2, id="never-seen")
    r3 = requests.post(url + "/v1/context/chat/completions", json=env3, headers=hh, timeout=timeout)
    code = None
    try:
        code = r3.json()["error"]["code"]
    except Exception:                                        # noqa: BLE001
        pass
    out.update(unknown_base=r3.status_code, unknown_base_code=code)
    out["ok"] = (key1 == chain_all(first) and out["ack"] == "v1" and out["stored"] == "1" and r2.status_code == 200
                 and out["stored_second"] == "3" and r3.status_code == 409 and code == "context_miss")
    return out


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
        ctx = context_check(url, h, report["models"][0], timeout)
        report["context"] = ctx
        ok = done and chunks > 0 and ctx["ok"]
    except Exception as e:                                   # noqa: BLE001 - a smoke test reports, it does not raise
        report["error"] = f"{type(e).__name__}: {e}"
        ok = False
    report["ok"] = ok
    print(json.dumps(report))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(run(*sys.argv[1:3]))

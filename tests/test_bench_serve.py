"""The synthetic serving sweep against the real HTTP front end over a socket (uvicorn in a thread, mock runner)."""
import socket
import threading
import time

import pytest

from ferrule_b200.server.bench_serve import _pct, run_sweep
from ferrule_b200.server.http import build_app

from test_server import make_worker


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.fixture()
def live_server():
    import uvicorn
    worker, runner = make_worker()
    port = _free_port()
    server = uvicorn.Server(uvicorn.Config(build_app(worker, "mock"), host="127.0.0.1", port=port, log_level="error"))
    thread = threading.Thread(target=server.run, daemon=True)
    thread.start()
    deadline = time.time() + 20
    while not server.started and time.time() < deadline:
        time.sleep(0.02)
    assert server.started, "uvicorn did not come up"
    yield f"http://127.0.0.1:{port}", worker
    server.should_exit = True
    thread.join(timeout=10)
    worker.stop()


def test_percentile_helper():
    assert _pct([], 0.5) == 0.0
    assert _pct([3.0, 1.0, 2.0], 0.5) == 2.0
    assert _pct([1.0, 2.0, 3.0, 4.0], 0.99) == 4.0


def test_sweep_counts_every_token_and_reads_server_counters(live_server):
    url, worker = live_server
    out = run_sweep(url, "mock", [1, 4], 6, seed=3, vocab=250, min_in=4, max_in=40, min_out=3, max_out=6, prefix=8,
                    frac=0.5)
    assert [lv["concurrency"] for lv in out["levels"]] == [1, 4]
    for lv in out["levels"]:
        assert lv["failed"] == 0 and lv["errors"] == []
        assert lv["requests"] == 6
        assert 6 * 3 <= lv["tokens"] <= 6 * 6             # ignore_eos: every request runs to its max_tokens
        assert lv["ttft_p50_s"] > 0 and lv["ttft_p99_s"] >= lv["ttft_p50_s"]
        assert lv["committed_tokens_per_s"] > 0
    srv = out["server"]
    assert srv["decode_steps"] > 0 and isinstance(srv["kv"], dict) and isinstance(srv["scheduler"], dict)
    assert worker.stats()["engine"]["decode_steps"] == srv["decode_steps"]


def test_sweep_raises_request_count_to_the_concurrency(live_server):
    url, _ = live_server
    out = run_sweep(url, "", [3], 1, seed=0, vocab=250, min_in=2, max_in=8, min_out=1, max_out=2, prefix=0, frac=0.0)
    assert out["levels"][0]["requests"] == 3 and out["levels"][0]["failed"] == 0


def test_sweep_reports_failures_instead_of_raising(live_server):
    url, _ = live_server
    # prompts beyond the context window are refused by the server: the sweep counts them and keeps the message
    out = run_sweep(url, "mock", [2], 3, seed=1, vocab=250, min_in=600, max_in=700, min_out=1, max_out=2, prefix=0,
                    frac=0.0)
    lv = out["levels"][0]
    assert lv["failed"] == 3 and lv["tokens"] == 0 and lv["errors"]


def test_sweep_against_a_dead_url_fails_every_request():
    out = run_sweep(f"http://127.0.0.1:{_free_port()}", "", [1], 2, seed=0, vocab=10, min_in=1, max_in=2, min_out=1,
                    max_out=1, prefix=0, frac=0.0)
    assert out["levels"][0]["failed"] == 2 and "unavailable" in out["server"]

"""HFStreamer / HTTPClient against a local http.server that speaks the hub's two routes."""
import http.server
import json
import os
import threading

import pytest

pa = pytest.importorskip("pyarrow")
import pyarrow.parquet as pq  # noqa: E402

from innova_b200.utils.hf_streamer import HFStreamer, HTTPClient  # noqa: E402


@pytest.fixture()
def hub(tmp_path):
    root = tmp_path / "hub"
    (root / "files").mkdir(parents=True)
    shards = [[f"doc {s}-{i}" for i in range(n)] for s, n in enumerate((5, 0, 7))]
    for s, rows in enumerate(shards):
        pq.write_table(pa.table({"text": rows, "id": list(range(len(rows)))}), root / "files" / f"{s}.parquet", row_group_size=3)
    (root / "files" / "broken.parquet").write_bytes(b"not parquet")
    listing = {"default": {"train": ["/files/0.parquet", "/files/broken.parquet", "/files/1.parquet", "/files/2.parquet"], "test": []}}
    seen = {"auth": [], "ranges": []}

    class H(http.server.SimpleHTTPRequestHandler):
        def __init__(self, *a, **k):
            super().__init__(*a, directory=str(root), **k)

        def log_message(self, *a):
            pass

        def do_GET(self):
            seen["auth"].append(self.headers.get("Authorization"))
            if self.path == "/api/datasets/org/data/parquet":
                body = json.dumps(listing).encode()
                self.send_response(200)
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)
                return
            rng = self.headers.get("Range")
            if rng and self.path.startswith("/files/"):
                seen["ranges"].append(rng)
                data = (root / self.path.lstrip("/")).read_bytes()
                lo, hi = rng.split("=")[1].split("-")
                lo = int(lo)
                hi = int(hi) if hi else len(data) - 1
                if lo >= len(data):
                    self.send_response(416)
                    self.end_headers()
                    return
                part = data[lo:hi + 1]
                self.send_response(206)
                self.send_header("Content-Length", str(len(part)))
                self.end_headers()
                self.wfile.write(part)
                return
            super().do_GET()

    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), H)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    yield f"http://127.0.0.1:{srv.server_address[1]}", shards, seen, root
    srv.shutdown()


def test_streams_every_row_of_every_readable_shard_in_order(hub, tmp_path):
    url, shards, seen, _ = hub
    st = HFStreamer(endpoint=url, cache_dir=str(tmp_path / "cache"))
    st.http.set_auth_token("tok")
    assert not st.is_open() and st.open("org/data", "train") and st.is_open()
    got = list(st)
    assert got == [r for rows in shards for r in rows] and st.samples_streamed() == 12
    assert "Bearer tok" in seen["auth"]
    assert os.listdir(tmp_path / "cache") == []                    # shards are dropped after use
    assert st.next_sample() is None
    st.close()
    assert not st.is_open()
    assert not st.open("org/data", "test") and not st.open("org/none", "train")     # empty split, unknown dataset


def test_http_client_ranges_length_and_resume(hub, tmp_path):
    url, _, seen, root = hub
    c = HTTPClient(retries=0)
    data = (root / "files" / "2.parquet").read_bytes()
    assert c.get_binary(url, "/files/2.parquet") == data
    assert c.range_request(url, "/files/2.parquet", 4, 19) == data[4:20]
    assert c.get_content_length(url, "/files/2.parquet") == len(data)
    assert json.loads(c.get(url, "/api/datasets/org/data/parquet"))["default"]["test"] == []
    dest = str(tmp_path / "x.parquet")
    open(dest + ".part", "wb").write(data[:100])                   # an interrupted download
    c.download(url + "/files/2.parquet", dest)
    assert open(dest, "rb").read() == data and f"bytes=100-" in seen["ranges"]
    open(dest + ".part", "wb").write(data)                         # everything was already there
    os.remove(dest)
    c.download(url + "/files/2.parquet", dest)
    assert open(dest, "rb").read() == data
    with pytest.raises(Exception):
        c.get(url, "/files/missing")

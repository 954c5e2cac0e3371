"""Streaming text samples of a Hugging Face dataset over HTTP: the Linux counterpart of the reference's ``HTTPClient`` /
``HFStreamer`` (include/oil/hf_streamer.h:36-81; its implementation is WinHTTP / ``_popen`` based, src/hf_streamer.cpp:180-260).

``HTTPClient``: ``get`` / ``get_binary`` / ``range_request`` / ``get_content_length`` with an optional bearer token, retries
with back-off, plain ``urllib``. ``HFStreamer.open(dataset, split)`` asks the hub for the dataset's auto-converted Parquet
shards (``/api/datasets/<name>/parquet``: ``{config: {split: [url, ...]}}``), then ``next_sample`` walks the shards in order:
a shard is fetched into a cache directory (resuming a partial file with a range request), read row group by row group
with ``ParquetStreamer`` and dropped again unless ``keep_shards`` is set. ``endpoint`` points anywhere that speaks the same
two routes, which is how the tests run it against a local ``http.server``. Nothing here needs a GPU.
"""
from __future__ import annotations

import json
import os
import tempfile
import time
import urllib.error
import urllib.parse
import urllib.request
from typing import List, Optional


class HTTPClient:
    def __init__(self, timeout: float = 30.0, retries: int = 3, backoff: float = 0.5):
        self.auth_token = ""
        self.timeout, self.retries, self.backoff = timeout, retries, backoff

    def set_auth_token(self, token: str):
        self.auth_token = token

    def _url(self, host: str, path: str, https: bool) -> str:
        if host.startswith("http://") or host.startswith("https://"):
            return host.rstrip("/") + path
        return ("https://" if https else "http://") + host + path

    def _open(self, url: str, headers=None, method: str = "GET"):
        h = {"User-Agent": "innova-b200/hf-streamer"}
        if self.auth_token:
            h["Authorization"] = "Bearer " + self.auth_token
        h.update(headers or {})
        last = None
        for attempt in range(self.retries + 1):
            try:
                return urllib.request.urlopen(urllib.request.Request(url, headers=h, method=method), timeout=self.timeout)
            except urllib.error.HTTPError as e:
                if e.code < 500 and e.code != 429:          # the request itself is wrong: no point in retrying
                    raise
                last = e
            except (urllib.error.URLError, TimeoutError, ConnectionError) as e:
                last = e
            time.sleep(self.backoff * (2 ** attempt))
        raise last

    def get(self, host: str, path: str, https: bool = True) -> str:
        with self._open(self._url(host, path, https)) as r:
            return r.read().decode("utf-8", "replace")

    def get_binary(self, host: str, path: str, https: bool = True) -> bytes:
        with self._open(self._url(host, path, https)) as r:
            return r.read()

    def range_request(self, host: str, path: str, start: int, end: int, https: bool = True) -> bytes:
        """Bytes [start, end] inclusive (the HTTP convention the reference uses)."""
        with self._open(self._url(host, path, https), {"Range": f"bytes={start}-{end}"}) as r:
            data = r.read()
            return data if r.status == 206 else data[start:end + 1]      # a server without range support sent everything

    def get_content_length(self, host: str, path: str, https: bool = True) -> int:
        with self._open(self._url(host, path, https), method="HEAD") as r:
            return int(r.headers.get("Content-Length", -1))

    def download(self, url: str, dest: str, chunk: int = 1 << 20) -> str:
        """Fetch ``url`` into ``dest``; a partial ``dest + '.part'`` from an earlier attempt is continued with a range request."""
        part = dest + ".part"
        have = os.path.getsize(part) if os.path.exists(part) else 0
        headers = {"Range": f"bytes={have}-"} if have else {}
        try:
            r = self._open(url, headers)
        except urllib.error.HTTPError as e:
            if e.code != 416:                                # 416: the part file already holds everything
                raise
            os.replace(part, dest)
            return dest
        with r:
            mode = "ab" if have and r.status == 206 else "wb"
            with open(part, mode) as f:
                while True:
                    buf = r.read(chunk)
                    if not buf:
                        break
                    f.write(buf)
        os.replace(part, dest)
        return dest


class HFStreamer:
    def __init__(self, endpoint: str = "https://huggingface.co", cache_dir: Optional[str] = None, text_column: str = "text",
                 config: Optional[str] = None, keep_shards: bool = False, client: Optional[HTTPClient] = None):
        self.endpoint = endpoint.rstrip("/")
        self.cache_dir = cache_dir or os.path.join(tempfile.gettempdir(), "innova_hf_cache")
        self.text_column, self.config, self.keep_shards = text_column, config, keep_shards
        self.http = client or HTTPClient()
        self._open_ = False
        self.samples_streamed_ = 0
        self.shard_urls: List[str] = []
        self._shard = -1
        self._rows: List[str] = []
        self._reader = None
        self._path: Optional[str] = None
        self.dataset_name = self.split = ""

    # ---- the reference's surface
    def open(self, dataset_name: str, split: str = "train") -> bool:
        self.close()
        self.dataset_name, self.split = dataset_name, split
        try:
            listing = json.loads(self.http.get(self.endpoint, "/api/datasets/" + urllib.parse.quote(dataset_name, safe="/") + "/parquet"))
        except Exception:                                    # noqa: BLE001 - an unreachable hub or unknown dataset is reported, not raised
            return False
        configs = listing if isinstance(listing, dict) else {}
        cfg = self.config if self.config in configs else (next(iter(configs)) if configs else None)
        urls = configs.get(cfg, {}).get(split, []) if cfg is not None else []
        if not urls:
            return False
        self.shard_urls = [u if "://" in u else self.endpoint + u for u in urls]
        os.makedirs(self.cache_dir, exist_ok=True)
        self._open_, self._shard, self.samples_streamed_ = True, -1, 0
        return True

    def is_open(self) -> bool:
        return self._open_

    def samples_streamed(self) -> int:
        return self.samples_streamed_

    def next_sample(self) -> Optional[str]:
        """The next text row, or None at the end of the split (the reference returns false and leaves ``text`` alone)."""
        while self._open_:
            if self._rows:
                self.samples_streamed_ += 1
                return self._rows.pop()
            if self._reader is not None and self._next_group():
                continue
            if not self._next_shard():
                return None
        return None

    def close(self):
        self._drop_shard()
        self._open_ = False
        self.shard_urls = []

    def __iter__(self):
        while True:
            s = self.next_sample()
            if s is None:
                return
            yield s

    # ---- shards
    def _drop_shard(self):
        self._reader, self._rows = None, []
        if self._path and not self.keep_shards and os.path.exists(self._path):
            os.remove(self._path)
        self._path = None

    def _next_shard(self) -> bool:
        import pyarrow.parquet as pq
        self._drop_shard()
        while self._shard + 1 < len(self.shard_urls):
            self._shard += 1
            url = self.shard_urls[self._shard]
            name = f"{self.dataset_name.replace('/', '--')}--{self.split}--{self._shard:05d}.parquet"
            dest = os.path.join(self.cache_dir, name)
            try:
                if not os.path.exists(dest):
                    self.http.download(url, dest)
                f = pq.ParquetFile(dest)
            except Exception:                                # noqa: BLE001 - a missing or damaged shard is skipped
                if os.path.exists(dest):
                    os.remove(dest)
                continue
            if self.text_column not in f.schema_arrow.names:
                if not self.keep_shards:
                    os.remove(dest)
                continue
            self._reader, self._group, self._path = f, 0, dest
            return True
        return False

    def _next_group(self) -> bool:
        f = self._reader
        if self._group >= f.num_row_groups:
            self._reader = None
            return False
        rows = f.read_row_group(self._group, columns=[self.text_column]).column(0).to_pylist()
        self._group += 1
        self._rows = [r for r in reversed(rows) if isinstance(r, str)]
        return True

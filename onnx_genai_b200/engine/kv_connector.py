"""KV offload connector: keep the K/V of finished prompts outside the device and bring it back on a prefix hit.

The device prefix cache only remembers what still fits in the page pool.  A connector extends it downwards: when a
request finishes, its K/V is stored in chunks of 256 tokens (16 pages) keyed by a chained hash of the token ids; when
a new request arrives, the longest run of leading chunks found in the connector is copied back into freshly adopted
pages and registered with the device prefix cache, so the scheduler admits the request as a prefix hit and only
computes the rest.  Same contract as the reference's ``KvCacheConnector`` (store / lookup / fetch / evict over
256-token chunks, crates/onnx-genai-kv/src/connector.rs:29-35) and its tiered local implementation with an
in-memory hot tier and a disk backing store (src/local_tiered.rs, src/backing_store.rs:62-130).

``LocalTieredConnector`` holds chunks in host memory up to ``max_host_bytes`` (least recently used chunks fall to
disk) and on disk up to ``max_disk_bytes`` (least recently used files are deleted).  Files are written to a
temporary name and renamed, so a crash never leaves a partial chunk under a valid key.
"""
from __future__ import annotations

import hashlib
import os
import threading
from collections import OrderedDict

import numpy as np
import torch

CHUNK_TOKENS = 256
PAGE_TOKENS = 16
PAGES_PER_CHUNK = CHUNK_TOKENS // PAGE_TOKENS


def chunk_keys(tokens, model_tag: str = "") -> list:
    """One key per full 256-token chunk of ``tokens``; each key covers the whole prefix up to its chunk."""
    arr = np.ascontiguousarray(tokens, dtype=np.int32)
    keys, h = [], hashlib.sha1(model_tag.encode()).digest()
    for c in range(len(arr) // CHUNK_TOKENS):
        h = hashlib.sha1(h + arr[c * CHUNK_TOKENS:(c + 1) * CHUNK_TOKENS].tobytes()).digest()
        keys.append(h.hex())
    return keys


class KvConnector:
    """Interface.  Values are opaque byte strings (one chunk of every layer's pages)."""

    def contains(self, key: str) -> bool:
        raise NotImplementedError

    def store(self, key: str, blob: bytes) -> None:
        raise NotImplementedError

    def fetch(self, key: str):
        raise NotImplementedError

    def evict(self, key: str) -> None:
        raise NotImplementedError


class LocalTieredConnector(KvConnector):
    def __init__(self, disk_dir: str | None = None, max_host_bytes: int = 1 << 30, max_disk_bytes: int = 8 << 30):
        self.host: OrderedDict = OrderedDict()
        self.host_bytes = 0
        self.max_host_bytes = max_host_bytes
        self.disk_dir = disk_dir
        self.max_disk_bytes = max_disk_bytes
        self.disk: OrderedDict = OrderedDict()      # key -> size, LRU order
        self.disk_bytes = 0
        self.lock = threading.Lock()
        self.stats = {"stores": 0, "host_hits": 0, "disk_hits": 0, "misses": 0, "spilled": 0, "deleted": 0}
        self.on_host_bytes = None       # callback(bytes now held in host memory), set by whoever accounts for them
        if disk_dir:
            os.makedirs(disk_dir, exist_ok=True)
            for name in sorted(os.listdir(disk_dir)):      # chunks written by an earlier process are usable again
                if name.endswith(".kv"):
                    size = os.path.getsize(os.path.join(disk_dir, name))
                    self.disk[name[:-3]] = size
                    self.disk_bytes += size

    def _path(self, key):
        return os.path.join(self.disk_dir, key + ".kv")

    def contains(self, key):
        with self.lock:
            return key in self.host or key in self.disk

    def store(self, key, blob):
        with self.lock:
            if key in self.host:
                self.host.move_to_end(key)
                return
            self.stats["stores"] += 1
            self.host[key] = blob
            self.host_bytes += len(blob)
            while self.host_bytes > self.max_host_bytes and len(self.host) > 1:
                old_key, old = self.host.popitem(last=False)
                self.host_bytes -= len(old)
                self._spill(old_key, old)
            held = self.host_bytes
        if self.on_host_bytes is not None:
            self.on_host_bytes(held)

    def _spill(self, key, blob):
        if not self.disk_dir or key in self.disk:
            return
        tmp = self._path(key) + ".tmp"
        with open(tmp, "wb") as f:
            f.write(blob)
        os.replace(tmp, self._path(key))
        self.disk[key] = len(blob)
        self.disk_bytes += len(blob)
        self.stats["spilled"] += 1
        while self.disk_bytes > self.max_disk_bytes and len(self.disk) > 1:
            old_key, size = self.disk.popitem(last=False)
            self.disk_bytes -= size
            self.stats["deleted"] += 1
            try:
                os.remove(self._path(old_key))
            except OSError:
                pass

    def shrink_host(self, nbytes: int) -> int:
        """Move least recently used chunks from host memory to disk (or drop them without a disk tier) until ``nbytes`` are
        free again; returns the bytes released.  The memory ledger calls this when another consumer of host memory is short."""
        freed = 0
        with self.lock:
            while freed < nbytes and self.host:
                key, blob = self.host.popitem(last=False)
                self.host_bytes -= len(blob)
                freed += len(blob)
                self._spill(key, blob)
        if self.on_host_bytes is not None:
            self.on_host_bytes(self.host_bytes)
        return freed

    def fetch(self, key):
        with self.lock:
            blob = self.host.get(key)
            if blob is not None:
                self.host.move_to_end(key)
                self.stats["host_hits"] += 1
                return blob
            if key in self.disk:
                try:
                    with open(self._path(key), "rb") as f:
                        blob = f.read()
                except OSError:
                    self.disk_bytes -= self.disk.pop(key)
                    self.stats["misses"] += 1
                    return None
                self.disk.move_to_end(key)
                self.stats["disk_hits"] += 1
                return blob
            self.stats["misses"] += 1
            return None

    def evict(self, key):
        with self.lock:
            blob = self.host.pop(key, None)
            if blob is not None:
                self.host_bytes -= len(blob)
            size = self.disk.pop(key, None)
            if size is not None:
                self.disk_bytes -= size
                try:
                    os.remove(self._path(key))
                except OSError:
                    pass

    def flush(self):
        """Write every host-resident chunk to disk (shutdown, or before handing the directory to another process)."""
        with self.lock:
            for key, blob in list(self.host.items()):
                self._spill(key, blob)


class KvOffload:
    """Glue between an :class:`LLMEngine` and a connector."""

    def __init__(self, llm, connector: KvConnector, model_tag: str = ""):
        self.llm, self.connector = llm, connector
        kv = llm.kv
        self.tag = model_tag or f"{llm.cfg.model.name}/{llm.cfg.kv_dtype}/L{len(kv.pools)}/{tuple(kv.pools[0].shape[1:])}/tp{llm.tp}r{llm.rank}"
        self.page_bytes = kv.pools[0][0].numel() * kv.pools[0].element_size()
        self.scale_bytes = kv.scales[0][0].numel() * 4 if kv.scales is not None else 0
        self.chunks_stored = 0
        self.chunks_restored = 0
        self.tokens_restored = 0

    # -- device -> connector --------------------------------------------------------------------
    def save(self, tokens) -> int:
        """Store every full chunk of ``tokens`` whose pages are in the device prefix cache (a request that just
        finished has published them) and that the connector does not hold yet; returns chunks stored."""
        toks = np.ascontiguousarray(tokens, dtype=np.int32)
        pages = self.llm.core.prefix_peek(toks)
        keys = chunk_keys(toks[: len(pages) * PAGE_TOKENS], self.tag)
        stored = 0
        for c, key in enumerate(keys):
            if (c + 1) * PAGES_PER_CHUNK > len(pages) or self.connector.contains(key):
                continue
            idx = torch.from_numpy(pages[c * PAGES_PER_CHUNK:(c + 1) * PAGES_PER_CHUNK].astype(np.int64)).to(self.llm.device)
            parts = []
            for li, pool in enumerate(self.llm.kv.pools):
                raw_pool = pool.view(torch.uint8) if pool.element_size() == 1 else pool
                parts.append(raw_pool.index_select(0, idx).contiguous().view(torch.uint8).cpu().numpy().tobytes())
                if self.llm.kv.scales is not None:
                    parts.append(self.llm.kv.scales[li].index_select(0, idx).contiguous().cpu().numpy().tobytes())
            self.connector.store(key, b"".join(parts))
            stored += 1
        self.chunks_stored += stored
        return stored

    # -- connector -> device --------------------------------------------------------------------
    def restore(self, tokens) -> int:
        """Bring back the longest run of leading chunks of ``tokens`` that the connector holds; returns the number of
        tokens now served by the device prefix cache thanks to it.  Call before ``add_request``."""
        toks = np.ascontiguousarray(tokens, dtype=np.int32)
        usable = (len(toks) - 1) // CHUNK_TOKENS          # the last token always runs, as with the device cache
        keys = chunk_keys(toks[: usable * CHUNK_TOKENS], self.tag)
        blobs = []
        for key in keys:
            blob = self.connector.fetch(key)
            if blob is None:
                break
            blobs.append(blob)
        # a blob written by a different model layout ends the run: nothing after it is adopted
        per_layer = PAGES_PER_CHUNK * (self.page_bytes + self.scale_bytes)
        want = per_layer * len(self.llm.kv.pools)
        good = 0
        while good < len(blobs) and len(blobs[good]) == want:
            good += 1
        blobs = blobs[:good]
        if not blobs:
            return 0
        # Adoption publishes a page under its prefix hash before any byte of it is written, so every adopted page
        # must be filled below or leave the cache again.  When the pool runs out in the middle of a chunk the pages
        # of that partial chunk are taken back out (a later request must never attach to uninitialised K/V).
        adopted = self.llm.core.prefix_adopt(toks[: len(blobs) * CHUNK_TOKENS])
        n_chunks = len(adopted) // PAGES_PER_CHUNK
        tail = adopted[n_chunks * PAGES_PER_CHUNK:]
        if len(tail):
            self.llm.core.prefix_unpublish(tail)
        restored_tokens = 0
        for c in range(n_chunks):
            page_ids = adopted[c * PAGES_PER_CHUNK:(c + 1) * PAGES_PER_CHUNK]
            fill = np.flatnonzero(page_ids >= 0)
            if len(fill) == 0:
                continue                                  # the device cache already had this chunk
            blob = np.frombuffer(blobs[c], dtype=np.uint8)
            dst = torch.from_numpy(page_ids[fill].astype(np.int64)).to(self.llm.device)
            for li, pool in enumerate(self.llm.kv.pools):
                base = li * per_layer
                # one-byte pools are moved as plain bytes (index kernels do not take every 8-bit float type)
                raw_pool = pool.view(torch.uint8) if pool.element_size() == 1 else pool
                pg = torch.from_numpy(blob[base:base + PAGES_PER_CHUNK * self.page_bytes].copy()).view(raw_pool.dtype).view(
                    (PAGES_PER_CHUNK,) + tuple(pool.shape[1:]))
                raw_pool.index_copy_(0, dst, pg[torch.from_numpy(fill)].to(self.llm.device))
                if self.llm.kv.scales is not None:
                    sc = torch.from_numpy(blob[base + PAGES_PER_CHUNK * self.page_bytes:base + per_layer].copy()).view(torch.float32).view(
                        (PAGES_PER_CHUNK,) + tuple(self.llm.kv.scales[li].shape[1:]))
                    self.llm.kv.scales[li].index_copy_(0, dst, sc[torch.from_numpy(fill)].to(self.llm.device))
            self.chunks_restored += 1
            restored_tokens += len(fill) * PAGE_TOKENS
        self.tokens_restored += restored_tokens
        return restored_tokens

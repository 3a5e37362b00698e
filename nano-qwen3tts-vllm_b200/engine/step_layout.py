"""Layout of one engine step that mixes prompt portions and single decoded tokens.

Per token: id, the id before it in its sequence (-1 at a sequence's first token), position, batch row, cache slot.  Per batch row (a sequence in this step): where its tokens start in
the packed batch, the position of the first one (= tokens already cached), how many there are, its state slot and its
block table.  Everything is written with numpy into ONE pinned buffer and crosses PCIe as ONE copy; the kernels read
the device mirror, whose addresses never change (CUDA graphs of the decode step are captured over them).
Rows past the live ones are padding: slot -1 / length 0, skipped by every kernel."""
from __future__ import annotations

import numpy as np
import torch


class MixedStepLayout:
    TOKEN_FIELDS = ("tokens", "prev_tokens", "positions", "tok_seq", "slot_mapping", "want_rows")
    SEQ_FIELDS = ("seq_start", "seq_pos0", "seq_len", "seq_slot")
    RING = 4

    def __init__(self, max_tokens: int, max_seqs: int, max_blocks: int, device):
        self.max_tokens, self.max_seqs, self.max_blocks = max_tokens, max_seqs, max_blocks
        off, self.offsets = 0, {}
        for name in self.TOKEN_FIELDS:
            self.offsets[name] = (off, max_tokens)
            off += (max_tokens + 3) // 4 * 4
        for name in self.SEQ_FIELDS:
            self.offsets[name] = (off, max_seqs)
            off += (max_seqs + 3) // 4 * 4
        self.offsets["block_tables"] = (off, max_seqs * max_blocks)
        off += max_seqs * max_blocks
        self.numel = off
        self.dev = torch.zeros(off, dtype=torch.int32, device=device)
        self.hosts, self.events, self.cur = [], [], 0
        for _ in range(self.RING):
            h = torch.zeros(off, dtype=torch.int32)
            if torch.cuda.is_available():
                h = h.pin_memory()
            self.hosts.append(h)
            self.events.append(None)
        self.n_tokens = self.n_seqs = self.max_new = self.n_want = 0

    def _view(self, buf, name):
        o, n = self.offsets[name]
        v = buf[o:o + n]
        return v.reshape(self.max_seqs, self.max_blocks) if name == "block_tables" else v

    def fill(self, items, page: int, want_rows=None, pad_seqs: int | None = None):
        """``items`` = [(sequence, tokens to run)].  ``want_rows``: packed-batch rows whose logits are wanted.
        ``pad_seqs``: lay the step out as exactly this many one-token rows (graph replay), padding the tail."""
        self.cur = (self.cur + 1) % self.RING
        if self.events[self.cur] is not None:
            self.events[self.cur].synchronize()
        host = self.hosts[self.cur]
        hn = host.numpy()
        f = {name: self._view(hn, name) for name in self.offsets}
        n_tok = sum(n for _, n in items)
        if n_tok > self.max_tokens or len(items) > self.max_seqs:
            raise RuntimeError(f"step of {n_tok} tokens / {len(items)} sequences exceeds the layout "
                               f"({self.max_tokens} / {self.max_seqs})")
        o = 0
        for b, (seq, n) in enumerate(items):
            c = seq.num_cached_tokens
            nb = len(seq.block_table)
            if nb > self.max_blocks:
                raise RuntimeError(f"sequence of {c + n} tokens exceeds max_model_len")
            ar = np.arange(c, c + n, dtype=np.int64)
            bt = np.asarray(seq.block_table, dtype=np.int64)
            f["tokens"][o:o + n] = seq.token_ids[c:c + n]
            # the token before each one: part of the sequence's state, so a portion's first token finds its predecessor
            f["prev_tokens"][o:o + n] = seq.token_ids[c - 1:c + n - 1] if c > 0 else [-1] + seq.token_ids[0:n - 1]
            f["positions"][o:o + n] = ar
            f["tok_seq"][o:o + n] = b
            f["slot_mapping"][o:o + n] = bt[ar // page] * page + ar % page
            f["seq_start"][b], f["seq_pos0"][b], f["seq_len"][b], f["seq_slot"][b] = o, c, n, seq.state_slot
            f["block_tables"][b, :nb] = bt
            o += n
        n_seqs = len(items)
        if pad_seqs is not None and pad_seqs > n_seqs:
            assert o == n_seqs
            f["tokens"][o:pad_seqs] = 0
            f["prev_tokens"][o:pad_seqs] = -1
            f["positions"][o:pad_seqs] = 0
            f["tok_seq"][o:pad_seqs] = np.arange(o, pad_seqs)
            f["slot_mapping"][o:pad_seqs] = -1
            f["seq_start"][n_seqs:pad_seqs] = np.arange(o, pad_seqs)
            f["seq_pos0"][n_seqs:pad_seqs] = 0
            f["seq_len"][n_seqs:pad_seqs] = 0
            f["seq_slot"][n_seqs:pad_seqs] = 0
            n_seqs = o = pad_seqs
        if want_rows is None:
            want_rows = []
        f["want_rows"][:len(want_rows)] = want_rows
        self.dev.copy_(host, non_blocking=True)
        if torch.cuda.is_available():
            ev = self.events[self.cur] or torch.cuda.Event()
            ev.record()
            self.events[self.cur] = ev
        self.n_tokens, self.n_seqs, self.n_want = o, n_seqs, len(want_rows)
        self.max_new = max((n for _, n in items), default=0)
        self._bind()

    def _bind(self):
        """Device views of the live part, under the names the kernels' wrappers read."""
        nt, ns = self.n_tokens, self.n_seqs
        for name in self.TOKEN_FIELDS:
            setattr(self, name, self._view(self.dev, name)[:self.n_want if name == "want_rows" else nt])
        for name in self.SEQ_FIELDS:
            setattr(self, name, self._view(self.dev, name)[:ns])
        self.block_tables = self._view(self.dev, "block_tables")[:max(ns, 1)]

    def set_decode_shape(self, rows: int):
        """Views for a captured decode step of ``rows`` one-token sequences (contents come from ``fill``)."""
        self.n_tokens = self.n_seqs = rows
        self.max_new, self.n_want = 1, 0
        self._bind()

"""Host-side holder of one Llama-style block on one GPU: weights, KV caches and workspace in device
memory, `prefill` / `decode` through the C ABI (`catena_b200_llama_prefill`, `catena_b200_llama_decode`).

The reference has no such model; the block is composed from its stdlib programs (rmsnorm without gain,
the matmul cell rule, softmax with math.exp-approx, nn.silu — see include/catena_b200.h).  Arrays cross
this interface as bf16 BIT PATTERNS (numpy uint16), the same convention as `gemm-bf16-rc`.
"""
import ctypes as C

import numpy as np

WEIGHT_NAMES = ("embedding", "w_qkv", "w_o", "w_gate_up", "w_down")


class LlamaBlock:
    def __init__(self, hidden, n_heads, n_kv_heads, ffn, vocab, max_len, weights, batch, rope_base=10000.0):
        """weights: dict name -> uint16 array of the shapes documented in catena_llama_block_t."""
        from . import CatenaMem, LlamaBlockStruct, check, lib, upload
        shapes = {"embedding": (vocab, hidden), "w_qkv": ((n_heads + 2 * n_kv_heads) * 128, hidden),
                  "w_o": (hidden, n_heads * 128), "w_gate_up": (2 * ffn, hidden), "w_down": (hidden, ffn)}
        self._mems = {}
        for name in WEIGHT_NAMES:
            w = np.ascontiguousarray(weights[name], dtype=np.uint16)
            if w.shape != shapes[name]:
                raise ValueError(f"{name}: expected shape {shapes[name]}, got {w.shape}")
            self._mems[name] = upload(w)
        self.hidden, self.n_heads, self.n_kv_heads, self.ffn, self.vocab = hidden, n_heads, n_kv_heads, ffn, vocab
        self.max_len, self.batch, self.pos = max_len, batch, 0
        self.struct = LlamaBlockStruct(hidden, n_heads, n_kv_heads, ffn, vocab, max_len, *[self._mems[n].data for n in WEIGHT_NAMES],
                                       rope_base)
        cache_bytes = batch * n_kv_heads * max_len * 128 * 2
        self.k_cache, self.v_cache = CatenaMem(), CatenaMem()
        zeros = np.zeros(cache_bytes // 2, np.uint16)      # rows past the visible length must stay finite
        self.k_cache, self.v_cache = upload(zeros), upload(zeros)
        self._ws = None
        self._ws_tokens = 0
        self._L = lib()
        self._check = check

    def _workspace(self, tokens):
        from . import CatenaMem, free
        if self._ws is None or self._ws_tokens < tokens:
            if self._ws is not None:
                free(self._ws)
            need = self._L.catena_b200_llama_workspace_bytes(C.byref(self.struct), tokens)
            self._ws = CatenaMem()
            self._check(self._L.catena_b200_mem_alloc(need, C.byref(self._ws)), "workspace")
            self._ws_tokens = tokens
        return self._ws

    def prefill(self, ids, seq, download=True):
        """ids [batch * seq] -> output activations [batch * seq, hidden] (bf16 bits); positions 0..seq-1."""
        from . import CatenaMem, download as dl, free, upload
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        if ids.size != self.batch * seq:
            raise ValueError("prefill: ids must hold batch * seq tokens")
        ws = self._workspace(self.batch * seq)
        idm = upload(ids)
        out = CatenaMem()
        self._check(self._L.catena_b200_mem_alloc(self.batch * seq * self.hidden * 2, C.byref(out)), "out")
        try:
            self._check(self._L.catena_b200_llama_prefill(C.byref(self.struct), idm.data, self.batch, seq, self.k_cache.data,
                                                          self.v_cache.data, out.data, ws.data, ws.len), "llama_prefill")
            self.pos = seq
            return dl(out, np.uint16).reshape(self.batch * seq, self.hidden) if download else None
        finally:
            free(idm)
            free(out)

    def decode(self, ids):
        """One token per sequence at the current position -> [batch, hidden] (bf16 bits)."""
        from . import CatenaMem, download as dl, free, upload
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        if ids.size != self.batch:
            raise ValueError("decode: one id per sequence")
        ws = self._workspace(self.batch)
        idm = upload(ids)
        out = CatenaMem()
        self._check(self._L.catena_b200_mem_alloc(self.batch * self.hidden * 2, C.byref(out)), "out")
        try:
            self._check(self._L.catena_b200_llama_decode(C.byref(self.struct), idm.data, self.batch, self.pos, self.k_cache.data,
                                                         self.v_cache.data, out.data, ws.data, ws.len), "llama_decode")
            self.pos += 1
            return dl(out, np.uint16).reshape(self.batch, self.hidden)
        finally:
            free(idm)
            free(out)

    def caches(self):
        """(k_cache, v_cache) as [batch, n_kv_heads, max_len, 128] bf16 bit arrays."""
        from . import download as dl
        shape = (self.batch, self.n_kv_heads, self.max_len, 128)
        return dl(self.k_cache, np.uint16).reshape(shape), dl(self.v_cache, np.uint16).reshape(shape)

    def close(self):
        from . import free
        for m in list(self._mems.values()) + [self.k_cache, self.v_cache] + ([self._ws] if self._ws is not None else []):
            free(m)
        self._mems, self._ws = {}, None

"""Host-side mirror of the llama2 extension's ``TransformerGpu`` (CudaExtension.llm32.llama2/Files/
llama2_gpu.cpp: ``build`` :335-346, ``forward(token, pos)`` :32-111) over the C ABI.

``build`` reads an 'ak42' version-1 checkpoint exactly as ``read_checkpoint`` /
``memory_map_weights`` do (llama2_cpu.cpp:74-159; the GPU twins llama2_gpu.cpp:234-333), uploads the weights, and allocates caches, RoPE
tables and the workspace once.  ``forward`` is one call of ``mca_llama_forward`` (5-6 kernel
launches per layer, nothing on the host) followed by the copy of the logits to the host that the
reference also makes (llama2_gpu.cpp:108).  Unlike the reference, ``batch`` independent sequences
step together, and the weights and caches may be held as bf16.

torch is used for device memory and streams only; without the CUDA library nothing here runs.
"""
from __future__ import annotations

import ctypes as C
import struct
import warnings

import numpy as np

from . import _lib

_MAGIC = 0x616B3432
_HEADER_BYTES = 256
_MAX_SEQ_LEN = 20480  # read_checkpoint clamps seq_len, llama2_cpu.cpp:143-144


class McaLlamaConfig(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("dim", "hidden_dim", "n_layers", "n_heads", "n_kv_heads", "vocab_size", "seq_len")]


class McaLlamaWeights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("token_embedding_table", "rms_att_weight", "rms_ffn_weight", "rms_final_weight",
                                          "wq", "wk", "wv", "wo", "w1", "w2", "w3", "wcls")] + [("weights_bf16", C.c_int)]


class McaLlamaState(C.Structure):
    _fields_ = [("key_cache", C.c_void_p), ("value_cache", C.c_void_p), ("cache_is_bf16", C.c_int),
                ("freq_real", C.c_void_p), ("freq_imag", C.c_void_p), ("workspace", C.c_void_p),
                ("workspace_floats", C.c_int64)]


def read_checkpoint(path):
    """Parse an 'ak42' v1 checkpoint into (config dict, {name: float32 array view}).  Follows
    read_checkpoint and memory_map_weights, llama2_cpu.cpp:79-159."""
    with open(path, "rb") as f:
        head = f.read(_HEADER_BYTES)
    if len(head) < 37:
        raise ValueError("ERROR_FILE_INVALID: checkpoint shorter than its header")
    magic, version = struct.unpack_from("<Ii", head, 0)
    if magic != _MAGIC or version != 1:
        raise ValueError("ERROR_FILE_INVALID: not an 'ak42' version-1 checkpoint")
    dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, seq_len = struct.unpack_from("<7i", head, 8)
    shared = struct.unpack_from("<B", head, 36)[0]
    seq_len = min(seq_len, _MAX_SEQ_LEN)
    cfg = dict(dim=dim, hidden_dim=hidden_dim, n_layers=n_layers, n_heads=n_heads, n_kv_heads=n_kv_heads,
               vocab_size=vocab_size, seq_len=seq_len)
    hs = dim // n_heads
    kv_dim = n_kv_heads * hs
    data = np.memmap(path, dtype=np.float32, mode="r", offset=_HEADER_BYTES)
    shapes = [("rms_att_weight", (n_layers, dim)), ("rms_ffn_weight", (n_layers, dim)), ("rms_final_weight", (dim,)),
              ("token_embedding_table", (vocab_size, dim)), ("wq", (n_layers, dim, dim)), ("wk", (n_layers, kv_dim, dim)),
              ("wv", (n_layers, kv_dim, dim)), ("wo", (n_layers, dim, dim)), ("w1", (n_layers, hidden_dim, dim)),
              ("w2", (n_layers, dim, hidden_dim)), ("w3", (n_layers, hidden_dim, dim))]
    if not shared:
        shapes.append(("wcls", (vocab_size, dim)))
    w, o = {}, 0
    for name, shape in shapes:
        n = int(np.prod(shape, dtype=np.int64))
        if o + n > data.size:
            raise ValueError("ERROR_FILE_INVALID: checkpoint shorter than its configuration says")
        w[name] = data[o:o + n].reshape(shape)
        o += n
    if shared:
        w["wcls"] = w["token_embedding_table"]
    return cfg, w


class TransformerGpu:
    """``build(checkpoint)`` then ``forward(token, pos)`` -> logits, as the reference class."""

    def __init__(self, device=0, batch=1, weights_bf16=False, cache_bf16=False, max_seq_len=None, use_graph=False):
        import torch
        if not torch.cuda.is_available():
            raise RuntimeError("TransformerGpu needs a CUDA device: there is no CPU path")
        self._torch = torch
        self._lib = _lib.load()
        self.device = torch.device("cuda", device)
        self.batch = int(batch)
        self.weights_bf16, self.cache_bf16 = bool(weights_bf16), bool(cache_bf16)
        self.max_seq_len = max_seq_len
        self.use_graph = bool(use_graph)   # replay the step from one CUDA graph (small models are launch-bound)
        self._graph = None
        self.config = None

    # -- build ------------------------------------------------------------------------------
    def build(self, checkpoint_path):
        cfg, w = read_checkpoint(checkpoint_path)
        self.load_weights(cfg, w)

    def load_weights(self, cfg, w):
        """``w`` maps the checkpoint's names to host arrays (float32)."""
        torch = self._torch
        if self.max_seq_len:
            cfg = dict(cfg, seq_len=min(cfg["seq_len"], int(self.max_seq_len)))
        self.config = cfg
        self._graph = None
        hs = cfg["dim"] // cfg["n_heads"]
        kv_dim = cfg["n_kv_heads"] * hs
        wdt = torch.bfloat16 if self.weights_bf16 else torch.float32

        def up(a, dt=torch.float32):
            a = np.ascontiguousarray(a, np.float32)
            with warnings.catch_warnings():   # a memory-mapped checkpoint is read-only; it is only copied from
                warnings.simplefilter("ignore", UserWarning)
                host = torch.from_numpy(a)
            return host.to(self.device).to(dt).contiguous()

        t = {n: up(w[n]) for n in ("token_embedding_table", "rms_att_weight", "rms_ffn_weight", "rms_final_weight")}
        for n in ("wq", "wk", "wv", "wo", "w1", "w2", "w3"):
            t[n] = up(w[n], wdt)
        shared = w["wcls"] is w["token_embedding_table"]
        t["wcls"] = t["token_embedding_table"] if (shared and not self.weights_bf16) else up(w["wcls"], wdt)
        self._t = t
        B, S, L = self.batch, cfg["seq_len"], cfg["n_layers"]
        cdt = torch.bfloat16 if self.cache_bf16 else torch.float32
        self.key_cache = torch.zeros(L, B, S, kv_dim, device=self.device, dtype=cdt)
        self.value_cache = torch.zeros(L, B, S, kv_dim, device=self.device, dtype=cdt)
        fr, fi = np.empty((S, hs // 2), np.float32), np.empty((S, hs // 2), np.float32)
        fp = C.POINTER(C.c_float)
        rc = self._lib.mca_rope_tables_host(S, hs, 10000.0, fr.ctypes.data_as(fp), fi.ctypes.data_as(fp))
        if rc:
            raise RuntimeError(f"mca_rope_tables_host failed with {rc}")
        self.freq_real, self.freq_imag = up(fr), up(fi)
        self._cfg_c = McaLlamaConfig(**cfg)
        need = self._lib.mca_llama_workspace_floats(C.byref(self._cfg_c), B, S)
        if need < 0:
            raise ValueError("configuration not supported (heads must divide dim, kv heads must divide heads)")
        self.workspace = torch.empty(need, device=self.device)
        self.logits = torch.empty(B, cfg["vocab_size"], device=self.device)
        self._tokens = torch.zeros(B, dtype=torch.int32, device=self.device)
        self._pos = torch.zeros(B, dtype=torch.int32, device=self.device)
        self._w_c = McaLlamaWeights(*[t[n].data_ptr() for n in ("token_embedding_table", "rms_att_weight",
                                                                 "rms_ffn_weight", "rms_final_weight", "wq", "wk", "wv",
                                                                 "wo", "w1", "w2", "w3", "wcls")],
                                    int(self.weights_bf16))
        self._s_c = McaLlamaState(self.key_cache.data_ptr(), self.value_cache.data_ptr(), int(self.cache_bf16),
                                  self.freq_real.data_ptr(), self.freq_imag.data_ptr(), self.workspace.data_ptr(),
                                  self.workspace.numel())

    # -- forward ----------------------------------------------------------------------------
    def enqueue(self, max_len, stream=None):
        """Enqueue one step on ``stream`` reading the device-side token and position arrays."""
        torch = self._torch
        st = stream if stream is not None else torch.cuda.current_stream(self.device)
        rc = self._lib.mca_llama_forward(C.byref(self._cfg_c), C.byref(self._w_c), C.byref(self._s_c),
                                         self._tokens.data_ptr(), self._pos.data_ptr(), self.batch, int(max_len),
                                         self.logits.data_ptr(), st.cuda_stream)
        if rc:
            raise RuntimeError(f"mca_llama_forward failed with {rc}")

    def _capture(self):
        """One graph serves every token: tokens and positions are read from device memory, and the
        split plan is the one for the longest sequence the cache holds (splits beyond a sequence's
        length return at once)."""
        torch = self._torch
        side = torch.cuda.Stream(self.device)
        graph = torch.cuda.CUDAGraph()
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            graph.capture_begin()
            self.enqueue(self.config["seq_len"], stream=side)
            graph.capture_end()
        torch.cuda.current_stream(self.device).wait_stream(side)
        self._graph = graph

    def forward_batch(self, tokens, pos):
        """tokens, pos: ``batch`` ints each -> logits (batch, vocab_size) on the host."""
        torch = self._torch
        if self.config is None:
            raise RuntimeError("build() has not been called")
        tokens = np.asarray(tokens, np.int32).reshape(self.batch)
        pos = np.asarray(pos, np.int32).reshape(self.batch)
        if pos.min() < 0 or pos.max() >= self.config["seq_len"]:
            raise ValueError("position outside the cache")
        with torch.cuda.device(self.device):
            self._tokens.copy_(torch.from_numpy(tokens))
            self._pos.copy_(torch.from_numpy(pos))
            if self._graph is not None:
                self._graph.replay()
            else:
                self.enqueue(int(pos.max()) + 1)     # also the warm-up that precedes a capture
                if self.use_graph:
                    result = self.logits.cpu().numpy()
                    self._capture()
                    return result
            result = self.logits.cpu().numpy()     # synchronises
            if self.batch > 8:
                # above eight sequences the projections run on the tensor cores: a bounded wait that gave up there
                # leaves stale logits and a status word
                st = (C.c_int * 4)()
                if self._lib.mca_proj_tc_status(st) == 0 and st[0] != 0:
                    raise RuntimeError(f"projection kernel gave up: status {list(st)}")
            return result

    def forward(self, token, pos):
        """The reference's signature: one sequence, logits (vocab_size) on the host."""
        if self.batch != 1:
            raise ValueError("forward(token, pos) is the batch-1 call; use forward_batch")
        return self.forward_batch([token], [pos])[0]

"""CPU oracle for the attention hot path.  TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the CPU-baseline / reference legs of the
benchmark import this package, and only as the checker.  The shipped package
(``mycaffe_b200``) never does.

Two shared objects sit behind it (built by ``oracle/Makefile``):

* ``_build/liboracle.so`` -- the CPU restatement in ``attn_oracle.cpp``;
* ``_ref/libllama2_ref.so`` -- the reference's own ``llama2_cpu.cpp`` compiled from the
  reference tree with the shim headers in ``ref_shim/`` (decode path only).
"""
from __future__ import annotations

import ctypes as C
import os
import struct
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB = None
_REF = None

_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(dtype=np.float64, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")


def build(force: bool = False) -> None:
    """Compile the checkers (make -C oracle).  The reference twin is only rebuilt when
    the reference tree is present; otherwise a prebuilt one is kept."""
    so, src = _HERE / "_build" / "liboracle.so", _HERE / "attn_oracle.cpp"
    stale = so.exists() and so.stat().st_mtime < src.stat().st_mtime
    if force or stale or not so.exists() or not (_HERE / "_ref" / "libllama2_ref.so").exists():
        cmd = ["make", "-C", str(_HERE)] + (["-B"] if force else [])
        ref = reference_root()
        if ref is not None:
            cmd.append(f"REFERENCE={ref}")
        subprocess.run(cmd, check=True, stdout=subprocess.DEVNULL)


def reference_root():
    """Where the reference's source tree is: $MYCAFFE_REFERENCE, else a directory named `reference` beside this
    repository; None when neither exists (the twin is then not rebuilt)."""
    cand = os.environ.get("MYCAFFE_REFERENCE")
    for c in ([Path(cand)] if cand else []) + [_HERE.parent.parent / "reference"]:
        if (c / "CudaExtension.llm32.llama2" / "Files" / "llama2_cpu.cpp").exists():
            return c
    return None


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        path = _HERE / "_build" / "liboracle.so"
        if not path.exists() or path.stat().st_mtime < (_HERE / "attn_oracle.cpp").stat().st_mtime:
            build()
        _LIB = C.CDLL(str(path))
        _LIB.oracle_num_threads.restype = C.c_int
    return _LIB


def ref_lib() -> C.CDLL | None:
    """The compiled reference twin, or None when it was never built."""
    global _REF
    if _REF is None:
        path = _HERE / "_ref" / "libllama2_ref.so"
        if not path.exists():
            return None
        _REF = C.CDLL(str(path))
        _REF.ref_llama_create.restype = C.c_void_p
        _REF.ref_llama_create.argtypes = [C.c_char_p, C.POINTER(C.c_long)]
        _REF.ref_llama_forward.restype = C.POINTER(C.c_float)
        _REF.ref_llama_forward.argtypes = [C.c_void_p, C.c_int, C.c_int]
        _REF.ref_llama_state.restype = C.POINTER(C.c_float)
        _REF.ref_llama_state.argtypes = [C.c_void_p, C.c_int]
        _REF.ref_llama_config.argtypes = [C.c_void_p, C.POINTER(C.c_int)]
        _REF.ref_llama_destroy.argtypes = [C.c_void_p]
    return _REF


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_num_threads(n: int | None = None) -> int:
    """Set the OpenMP team size of the checkers (this library and the compiled reference twin share the
    runtime).  Default: every core this process may run on.  Returns the size now in effect."""
    if n is None:
        try:
            n = len(os.sched_getaffinity(0))
        except AttributeError:
            n = os.cpu_count() or 1
    lib().oracle_set_num_threads(int(n))
    return num_threads()


def _c(a, dt=np.float32):
    return np.ascontiguousarray(a, dtype=dt)


def _mask_args(mask, mask_mode):
    if mask_mode == 3:
        return np.zeros(1, np.float32), 3
    if mask is None or mask_mode == 0:
        return np.zeros(1, np.float32), 0
    return _c(mask), int(mask_mode)


# --------------------------------------------------------------------------- SDPA

def sdpa_forward(q, k, v, mask=None, mask_mode=0, f64=False, want_probs=False):
    """Reference SDPA forward (attn.cu:518-602).  q,k,v: (B,H,T,D) float32.
    mask_mode 1: (T,T) keep-mask; 2: (B,T) key keep-mask.  Returns y (and P)."""
    q, k, v = _c(q), _c(k), _c(v)
    B, H, T, D = q.shape
    m, mode = _mask_args(mask, mask_mode)
    dt = np.float64 if f64 else np.float32
    y = np.empty((B, H, T, D), dt)
    p = np.empty((B, H, T, T), dt) if want_probs else None
    fn = lib().oracle_sdpa_forward_f64 if f64 else lib().oracle_sdpa_forward_f32
    fn(q.ctypes, k.ctypes, v.ctypes, m.ctypes, mode, B, H, T, D, y.ctypes,
       p.ctypes if p is not None else None)
    return (y, p) if want_probs else y


def sdpa_forward_rows(q, k, v, mask, mask_mode, q_begin, q_step):
    """Forward for the query rows q_begin::q_step only (bounded work at long T)."""
    q, k, v = _c(q), _c(k), _c(v)
    B, H, T, D = q.shape
    m, mode = _mask_args(mask, mask_mode)
    y = np.zeros((B, H, T, D), np.float32)
    lib().oracle_sdpa_forward_rows_f32(q.ctypes, k.ctypes, v.ctypes, m.ctypes, mode, B, H, T, D, y.ctypes,
                                       int(q_begin), int(q_step))
    return y[:, :, q_begin::q_step]


def sdpa_backward(q, k, v, dy, mask=None, mask_mode=0, f64=False):
    """Reference SDPA backward (attn.cu:608-661).  Returns dq, dk, dv."""
    q, k, v, dy = _c(q), _c(k), _c(v), _c(dy)
    B, H, T, D = q.shape
    m, mode = _mask_args(mask, mask_mode)
    dt = np.float64 if f64 else np.float32
    dq, dk, dv = (np.empty((B, H, T, D), dt) for _ in range(3))
    fn = lib().oracle_sdpa_backward_f64 if f64 else lib().oracle_sdpa_backward_f32
    fn(q.ctypes, k.ctypes, v.ctypes, dy.ctypes, m.ctypes, mode, B, H, T, D, dq.ctypes, dk.ctypes, dv.ctypes)
    return dq, dk, dv


def causal_mask(T):
    """fillMask, CausalSelfAttentionLayer.cs:276-291: lower-triangular ones."""
    return np.tril(np.ones((T, T), np.float32))


# --------------------------------------------------------------------------- RoPE

def rope_tables(T, D, theta=10000.0):
    cos_t = np.empty((T, D // 2), np.float32)
    sin_t = np.empty((T, D // 2), np.float32)
    lib().oracle_rope_tables(int(T), int(D), C.c_float(theta), cos_t.ctypes, sin_t.ctypes)
    return cos_t, sin_t


def rope_apply(x, T, H, D, cos_t, sin_t, freq_offset=-1, backward=False):
    """RoPE on a (B,T,H,D) tensor (rope.cu:724-864)."""
    x = _c(x)
    y = np.empty_like(x)
    lib().oracle_rope_apply(x.ctypes, y.ctypes, C.c_int64(x.size), int(T), int(H), int(D),
                            _c(cos_t).ctypes, _c(sin_t).ctypes, int(freq_offset), int(bool(backward)))
    return y


# --------------------------------------------------------------------------- TFT

def tft_mask(num_hist, num_fut):
    """generate_mask (encoder-decoder form), MultiHeadAttentionInterpLayer.cs:306-327:
    1 marks a masked (future) key."""
    i = np.arange(num_fut)[:, None]
    j = np.arange(num_hist + num_fut)[None, :]
    return ((j > num_hist) & (j - num_hist > i)).astype(np.float32)


def tft_forward(q, k, v, mask=None, f64=False):
    """q (B,H,Nq,d), k (B,H,Nk,d), v (B,Nk,d) -> out (B,Nq,d), attn (B,Nq,Nk)."""
    q, k, v = _c(q), _c(k), _c(v)
    B, H, Nq, d = q.shape
    Nk = k.shape[2]
    dt = np.float64 if f64 else np.float32
    out = np.empty((B, Nq, d), dt)
    attn = np.empty((B, Nq, Nk), dt)
    fn = lib().oracle_tft_forward_f64 if f64 else lib().oracle_tft_forward_f32
    fn(q.ctypes, k.ctypes, v.ctypes, _c(mask).ctypes if mask is not None else None, B, H, Nq, Nk, d,
       out.ctypes, attn.ctypes)
    return out, attn


def tft_backward(q, k, v, mask, d_out, d_attn=None, f64=False):
    q, k, v, d_out = _c(q), _c(k), _c(v), _c(d_out)
    B, H, Nq, d = q.shape
    Nk = k.shape[2]
    dt = np.float64 if f64 else np.float32
    dq = np.empty((B, H, Nq, d), dt)
    dk = np.empty((B, H, Nk, d), dt)
    dv = np.empty((B, Nk, d), dt)
    fn = lib().oracle_tft_backward_f64 if f64 else lib().oracle_tft_backward_f32
    fn(q.ctypes, k.ctypes, v.ctypes, _c(mask).ctypes if mask is not None else None, d_out.ctypes,
       _c(d_attn).ctypes if d_attn is not None else None, B, H, Nq, Nk, d, dq.ctypes, dk.ctypes, dv.ctypes)
    return dq, dk, dv


# --------------------------------------------------------------------------- llama2 decode

def layernorm_forward(x, eps=1e-10):
    """LayerNormData<T>::Forward (layernorm.cu:291-333) over the last axis: returns (y, stdev)."""
    x = _c(x)
    rows, inner = int(np.prod(x.shape[:-1])), x.shape[-1]
    y, sd = np.empty_like(x), np.empty(rows, np.float32)
    lib().oracle_layernorm_fwd(x.ctypes, y.ctypes, sd.ctypes, C.c_int64(rows), inner, C.c_float(eps))
    return y, sd


def layernorm_backward(y, dy, stdev, eps=1e-10):
    """LayerNormData<T>::Backward (layernorm.cu:340-384), including its eps on the first `rows` elements."""
    y, dy, stdev = _c(y), _c(dy), _c(stdev)
    rows, inner = stdev.size, y.shape[-1]
    dx = np.empty_like(y)
    lib().oracle_layernorm_bwd(y.ctypes, dy.ctypes, stdev.ctypes, dx.ctypes, C.c_int64(rows), inner, C.c_float(eps))
    return dx


def rmsnorm_layer_forward(x, w=None, eps=1e-5):
    """RMSNormLayer<T>.forward (RMSNormLayer.cs:156-179) over the last axis: returns (y, 1/rms)."""
    x = _c(x)
    rows, inner = int(np.prod(x.shape[:-1])), x.shape[-1]
    y, inv = np.empty_like(x), np.empty(rows, np.float32)
    wc = _c(w) if w is not None else None
    lib().oracle_rmsnorm_layer_fwd(x.ctypes, wc.ctypes if wc is not None else None, y.ctypes, inv.ctypes, C.c_int64(rows),
                                   inner, C.c_float(eps))
    return y, inv


def rmsnorm_layer_backward(x, w, dy, eps=1e-5):
    """RMSNormLayer<T>.backward (RMSNormLayer.cs:190-231): returns (dx, dw); dw is None without weights."""
    x, dy = _c(x), _c(dy)
    rows, inner = int(np.prod(x.shape[:-1])), x.shape[-1]
    dx = np.empty_like(x)
    wc = _c(w) if w is not None else None
    dw = np.empty(inner, np.float32) if w is not None else None
    lib().oracle_rmsnorm_layer_bwd(x.ctypes, wc.ctypes if wc is not None else None, dy.ctypes, dx.ctypes,
                                   dw.ctypes if dw is not None else None, C.c_int64(rows), inner, C.c_float(eps))
    return dx, dw


def llama_freqs(head_size, seq_len, theta=10000.0):
    fr = np.empty((seq_len, head_size // 2), np.float32)
    fi = np.empty((seq_len, head_size // 2), np.float32)
    lib().oracle_llama_freqs(int(head_size), C.c_int64(seq_len), C.c_float(theta), fr.ctypes, fi.ctypes)
    return fr, fi


def rmsnorm(x, w, eps=1e-5):
    x, w = _c(x), _c(w)
    o = np.empty_like(x)
    lib().oracle_rmsnorm(o.ctypes, x.ctypes, w.ctypes, int(x.size), C.c_float(eps))
    return o


def gemv(w, x):
    w, x = _c(w), _c(x)
    d, n = w.shape
    out = np.empty(d, np.float32)
    lib().oracle_gemv(out.ctypes, x.ctypes, w.ctypes, int(n), int(d))
    return out


def llama_decode(q, k, v, key_cache, value_cache, pos, n_heads, n_kv_heads, theta=10000.0, want_att=False):
    """One decode step of the attention core for B independent sequences
    (llama2_cpu.cpp:290-342).  q (B,dim), k,v (B,kv_dim) are pre-RoPE; caches
    (B,seq_len,kv_dim) are updated in place at row pos[b].  Returns out (B,dim)."""
    q, k, v = _c(q).copy(), _c(k).copy(), _c(v)
    assert key_cache.dtype == np.float32 and key_cache.flags.c_contiguous
    assert value_cache.dtype == np.float32 and value_cache.flags.c_contiguous
    B, dim = q.shape
    hs = dim // n_heads
    seq_len = key_cache.shape[1]
    pos = _c(pos, np.int32)
    fr, fi = llama_freqs(hs, seq_len, theta)
    out = np.empty((B, dim), np.float32)
    att = np.zeros((B, n_heads, seq_len), np.float32) if want_att else None
    lib().oracle_llama_decode(q.ctypes, k.ctypes, v.ctypes, key_cache.ctypes, value_cache.ctypes, pos.ctypes,
                              B, int(n_heads), int(n_kv_heads), hs, seq_len, fr.ctypes, fi.ctypes, out.ctypes,
                              att.ctypes if att is not None else None)
    return (out, q, k, att) if want_att else out


def llama_forward(cfg, w, key_cache, value_cache, tokens, pos):
    """One whole-transformer decode step, token -> logits, for B independent sequences: the
    order of operations of TransformerCpu::forward (llama2_cpu.cpp:264-386) restated over the
    pieces above.  ``cfg`` has the reference's Config fields; ``w`` the checkpoint's arrays;
    caches (n_layers, B, seq_len, kv_dim) float32 are updated in place.  Unlike the compiled
    reference this also runs n_kv_heads < n_heads (its rope walks n_heads heads of the kv_dim-long
    k vector, llama2_cpu.cpp:243-246,293, which overruns the buffer)."""
    dim, L = cfg["dim"], cfg["n_layers"]
    tokens, pos = np.asarray(tokens).reshape(-1), _c(np.asarray(pos).reshape(-1), np.int32)
    B = tokens.size
    x = np.stack([_c(w["token_embedding_table"][int(t)]) for t in tokens]).copy()
    for l in range(L):
        q = np.empty((B, dim), np.float32)
        kv_dim = w["wk"].shape[1]
        k, v = np.empty((B, kv_dim), np.float32), np.empty((B, kv_dim), np.float32)
        for b in range(B):
            xb = rmsnorm(x[b], w["rms_att_weight"][l])
            q[b], k[b], v[b] = gemv(w["wq"][l], xb), gemv(w["wk"][l], xb), gemv(w["wv"][l], xb)
        att = llama_decode(q, k, v, key_cache[l], value_cache[l], pos, cfg["n_heads"], cfg["n_kv_heads"])
        for b in range(B):
            x[b] = x[b] + gemv(w["wo"][l], att[b])
            xb = rmsnorm(x[b], w["rms_ffn_weight"][l])
            hb, hb2 = gemv(w["w1"][l], xb), gemv(w["w3"][l], xb)
            hb = hb * (np.float32(1.0) / (np.float32(1.0) + np.exp(-hb))) * hb2
            x[b] = x[b] + gemv(w["w2"][l], hb)
    wcls = w.get("wcls", w["token_embedding_table"])
    return np.stack([gemv(wcls, rmsnorm(x[b], w["rms_final_weight"])) for b in range(B)])


def write_llama_checkpoint(path, dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, seq_len, weights):
    """Write a llama2.c 'ak42' version-1 checkpoint (read_checkpoint, llama2_cpu.cpp:108-159;
    weight order memory_map_weights :79-103).  ``weights`` maps names to float32 arrays."""
    order = ["rms_att_weight", "rms_ffn_weight", "rms_final_weight", "token_embedding_table",
             "wq", "wk", "wv", "wo", "w1", "w2", "w3"]
    with open(path, "wb") as f:
        f.write(struct.pack("<I", 0x616B3432))
        f.write(struct.pack("<i", 1))
        f.write(struct.pack("<7i", dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, seq_len))
        f.write(struct.pack("<B", 1))  # classifier shares the embedding table
        f.write(b"\0" * (256 - f.tell()))
        for name in order:
            f.write(np.ascontiguousarray(weights[name], np.float32).tobytes())


class RefLlama:
    """The reference's own TransformerCpu (compiled from its source) behind ctypes."""

    def __init__(self, checkpoint_path):
        r = ref_lib()
        if r is None:
            raise RuntimeError("oracle/_ref/libllama2_ref.so was not built")
        err = C.c_long(0)
        self._r = r
        self._h = r.ref_llama_create(os.fsencode(checkpoint_path), C.byref(err))
        if not self._h:
            raise RuntimeError(f"reference build() failed with {err.value}")
        cfg = (C.c_int * 7)()
        r.ref_llama_config(self._h, cfg)
        (self.dim, self.hidden_dim, self.n_layers, self.n_heads, self.n_kv_heads, self.vocab_size,
         self.seq_len) = list(cfg)

    def forward(self, token, pos):
        self._r.ref_llama_forward(self._h, int(token), int(pos))

    def state(self, name):
        idx = ["x", "xb", "xb2", "q", "k", "v", "att", "logits", "key_cache", "value_cache",
               "freq_real", "freq_imag"].index(name)
        kv_dim = self.dim * self.n_kv_heads // self.n_heads
        hs = self.dim // self.n_heads
        n = {"x": self.dim, "xb": self.dim, "xb2": self.dim, "q": self.dim, "k": kv_dim, "v": kv_dim,
             "att": self.n_heads * self.seq_len, "logits": self.vocab_size,
             "key_cache": self.n_layers * self.seq_len * kv_dim,
             "value_cache": self.n_layers * self.seq_len * kv_dim,
             "freq_real": self.seq_len * hs // 2, "freq_imag": self.seq_len * hs // 2}[name]
        ptr = self._r.ref_llama_state(self._h, idx)
        return np.ctypeslib.as_array(ptr, shape=(n,))

    def close(self):
        if self._h:
            self._r.ref_llama_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

"""The reference arm of bench.py: Leeaandrob/neurogrid's own CUDA library, unmodified, driven
through its stock C entry points from Python with ctypes.

The reference's LFM2 compute path is ``libgpu_engine.so`` (built by its own Makefile rule, see
``baseline/build_reference.sh``); its Go program around it cannot be built here (no Go
toolchain), so this file stands where ``pkg/inference`` stands in the reference and makes the
same calls in the same order:

* start-up          pkg/inference/engine_gpu.go:26-298, cuda_executor.go:182-231,546-590,742-794,1068-1097
* prefill           cuda_executor.go:307-419  ->  cuda_prefill_batch (gpu/engine/decode_all.cu:629-792)
* decode, 1 request batch_scheduler.go:421-557  ->  cuda_decode_step_gpu (decode_all.cu:509-603)
* decode, N > 1     batch_scheduler.go:250-418  ->  cuda_decode_step_batched (decode_all.cu:820-943)
* LM head           gpu_lmhead.go:229-290       ->  cuda_rmsnorm, cuda_gemm_fp16, cuda_copy_to_host
* sampling          sampler.go:58-73 (argmax on the host over float32 logits)

Nothing of neurogrid_b200 (and no torch) is imported: weights are drawn with numpy, device time
is taken with CUDA events through libcudart.  Limits of the reference that the caller has to
respect: nH * head_dim == hidden (its buffers are sized so, gpu/engine/layer.cu:1506,1539), a
context below 4,096 tokens (shared memory of its decode attention, gpu/cuda/paged_attention.cu:
577-578, and its 256-entry block table, cuda_executor.go:223).

Two numbers per batch size.  ``value``: device time of the model and LM-head calls of K decode
steps, the decode graph left to replay where the reference can replay it (one request): its best
case.  ``e2e``: the whole stock per-token sequence of its scheduler: conv states restored and
saved through the host, the graph invalidated, block tables and positions copied, logits copied
back as float32 and the argmax taken on the host.
"""
from __future__ import annotations

import ctypes as C
import os
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_ref", "libgpu_engine.so")
BLOCK = 16                     # pkg/inference/paged_kvcache.go:23
MAX_BLOCKS = 256               # cuda_executor.go:223
MAX_CONTEXT = 4000             # below the 4,096 scores its decode attention has shared memory for
VP = C.c_void_p


class Unavailable(RuntimeError):
    pass


def _bf16_bits(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


class _Pool:
    """Normal numbers drawn once; tensors take slices of them (distinct offsets per tensor)."""

    def __init__(self, seed: int, n: int = 1 << 26):
        self.rng = np.random.default_rng(seed)
        self.pool = self.rng.standard_normal(n, dtype=np.float32)

    def take(self, n: int, std: float, mean: float = 0.0) -> np.ndarray:
        if n > self.pool.size:
            reps = -(-n // self.pool.size)
            x = np.tile(self.pool, reps)[:n]
        else:
            at = int(self.rng.integers(0, self.pool.size - n + 1))
            x = self.pool[at:at + n]
        return x * np.float32(std) + np.float32(mean)

    def bf16(self, n, std, mean=0.0):
        return _bf16_bits(self.take(n, std, mean))

    def fp16(self, n, std, mean=0.0):
        # the reference turns bf16 checkpoints into fp16 for the embedding, the head and the final norm
        return self.take(n, std, mean).astype(np.float16)


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(VP)


class _Named:
    """Tensors of a model folder by their LFM2 names (numpy float32), handed out in the formats
    the reference uploads: bf16 bits for the layers, fp16 for the embedding, head and final norm."""

    def __init__(self, tensors: dict):
        self.t = tensors

    def bf16(self, name):
        return _bf16_bits(np.ascontiguousarray(self.t[name], dtype=np.float32).reshape(-1))

    def fp16(self, name):
        return np.ascontiguousarray(self.t[name], dtype=np.float32).reshape(-1).astype(np.float16)


class Reference:
    def __init__(self, cfg: dict, gpu: int = 0, max_batch: int = 8, seed: int = 0, tensors: dict = None):
        """``tensors``: float32 arrays by LFM2 tensor name (a model folder's weights); without them
        the weights are drawn from ``seed``."""
        if not os.path.isfile(LIB_PATH):
            raise Unavailable(f"{LIB_PATH} is not built (run baseline/build_reference.sh where nvcc is)")
        # the CUDA toolkit's runtime, the one the library was built with and has an rpath to
        cuda = os.environ.get("CUDA_PATH", "/usr/local/cuda")
        try:
            self.rt = C.CDLL(os.path.join(cuda, "lib64", "libcudart.so.12"), mode=C.RTLD_GLOBAL)
        except OSError:
            self.rt = C.CDLL("libcudart.so.12", mode=C.RTLD_GLOBAL)
        self.lib = C.CDLL(LIB_PATH)
        self._declare()
        H, I = cfg["hidden_size"], cfg["intermediate_size"]
        nH, nKV, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
        if nH * hd != H:
            raise Unavailable("the reference sizes its q buffers as hidden_size: it needs heads * head_dim == hidden")
        self.cfg, self.H, self.I, self.nH, self.nKV, self.hd = cfg, H, I, nH, nKV, hd
        self.V, self.K, self.eps = cfg["vocab_size"], cfg["conv_L_cache"], float(cfg["norm_eps"])
        self.types = [0 if t == "conv" else 1 for t in cfg["layer_types"]]
        self.max_batch = max_batch
        lib = self.lib
        self._ok(lib.cuda_init(gpu), "cuda_init")
        named = _Named(tensors) if tensors is not None else None
        pool = _Pool(seed) if named is None else None
        # embeddings, LM head (the tied table is uploaded a second time, engine_gpu.go:52-69), final norm
        table = pool.fp16(self.V * H, 0.02) if named is None else named.fp16("model.embed_tokens.weight")
        self.embed = self._upload(table)
        self.lm_head = self._upload(table if named is None or "lm_head.weight" not in named.t
                                    else named.fp16("lm_head.weight"))
        self.final_norm = self._upload(pool.fp16(H, 0.1, 1.0) if named is None
                                       else named.fp16("model.embedding_norm.weight"))
        self.hidden_gpu, self.normed_gpu = self._alloc(H * 2), self._alloc(H * 2)
        self.logits_gpu = self._alloc(self.V * 2)
        self.logits_host = np.empty(self.V, dtype=np.float32)
        # layers
        self.weights, self.conv_states, self.paged = [], {}, {}
        blocks = max_batch * MAX_BLOCKS
        for i, t in enumerate(self.types):
            w = VP()
            norm = lambda: pool.bf16(H, 0.1, 1.0)
            pre = f"model.layers.{i}."
            ffn_names = [pre + "feed_forward.w1.weight", pre + "feed_forward.w3.weight", pre + "feed_forward.w2.weight"]
            if t == 0:
                if named is not None:                            # pkg/model/loader.go:406-458
                    a = [named.bf16(pre + n) for n in ("conv.in_proj.weight", "conv.conv.weight", "conv.out_proj.weight",
                                                       "operator_norm.weight", "ffn_norm.weight")] + \
                        [named.bf16(n) for n in ffn_names]
                else:
                    a = [pool.bf16(3 * H * H, 0.02), pool.bf16(H * self.K, 0.2), pool.bf16(H * H, 0.02), norm(), norm(),
                         pool.bf16(I * H, 0.02), pool.bf16(I * H, 0.02), pool.bf16(H * I, 0.02)]
                self._ok(lib.cuda_create_conv_layer_weights_bf16(C.byref(w), *[_ptr(x) for x in a], H, I, self.K,
                                                                 self.eps), "conv layer weights")
                st = lib.cuda_conv_state_create(1, H, self.K)
                if not st:
                    raise Unavailable("cuda_conv_state_create failed")
                self.conv_states[i] = VP(st)
            else:
                kv = nKV * hd
                if named is not None:                            # pkg/model/loader.go:530-583
                    a = [named.bf16(pre + f"self_attn.{n}.weight") for n in ("q_proj", "k_proj", "v_proj", "out_proj")] + \
                        [named.bf16(n) for n in ffn_names] + \
                        [named.bf16(pre + n) for n in ("operator_norm.weight", "ffn_norm.weight",
                                                       "self_attn.q_layernorm.weight", "self_attn.k_layernorm.weight")]
                else:
                    a = [pool.bf16(H * H, 0.02), pool.bf16(kv * H, 0.02), pool.bf16(kv * H, 0.02), pool.bf16(H * H, 0.02),
                         pool.bf16(I * H, 0.02), pool.bf16(I * H, 0.02), pool.bf16(H * I, 0.02), norm(), norm(),
                         pool.bf16(hd, 0.1, 1.0), pool.bf16(hd, 0.1, 1.0)]
                self._ok(lib.cuda_create_layer_weights_bf16_native(C.byref(w), *[_ptr(x) for x in a], H, I, nH, nKV, hd),
                         "attention layer weights")
                pc = VP()
                self._ok(lib.cuda_paged_kvcache_create(C.byref(pc), blocks, nKV, hd, BLOCK), "paged cache")
                self.paged[i] = pc
            self.weights.append(w)
        del pool, table
        self.n_conv = len(self.conv_states)
        self.state_bytes = H * self.K * 4
        # workspaces, decode context (BuildDecodeContext + the paged and conv set-up of engine_gpu.go:245-276)
        self.ws, self.conv_ws, self.ctx = VP(), VP(), VP()
        self._ok(lib.cuda_create_layer_workspace_bf16(C.byref(self.ws), 1, H, I, nKV, hd), "bf16 workspace")
        self._ok(lib.cuda_create_decode_context(C.byref(self.ctx), len(self.types), H, I, nH, nKV, hd, self.eps,
                                                float(cfg["rope_theta"]), 1, self.K), "decode context")
        for i, t in enumerate(self.types):
            lib.cuda_set_decode_layer(self.ctx, i, t, self.weights[i], self.conv_states.get(i, VP()))
        self._ok(lib.cuda_set_decode_bf16_native(self.ctx, self.ws), "bf16 native mode")
        self.block_table_gpu = self._alloc(MAX_BLOCKS * 4)
        lib.cuda_set_decode_paged_cache(self.ctx, None, self.block_table_gpu, MAX_BLOCKS)
        for i, pc in self.paged.items():
            lib.cuda_set_decode_paged_layer(self.ctx, i, pc)
        self._ok(lib.cuda_create_conv_workspace(C.byref(self.conv_ws), H, I), "conv workspace")
        lib.cuda_set_decode_conv_workspace(self.ctx, self.conv_ws)
        # per request: its block table (blocks b*256 .. b*256+255 of every layer's pool), its position,
        # the host copy of its conv states (pkg/inference/sequence.go:20-47)
        self.tables = [np.arange(b * MAX_BLOCKS, (b + 1) * MAX_BLOCKS, dtype=np.int32) for b in range(max_batch)]
        self.position = [0] * max_batch
        self.saved = [dict() for _ in range(max_batch)]
        self.last_hidden = [None] * max_batch
        self.sync()

    # ------------------------------------------------------------------ plumbing
    def _declare(self):
        L, rt = self.lib, self.rt
        i, f, sz = C.c_int, C.c_float, C.c_size_t
        sig = {
            "cuda_init": [i], "cuda_malloc": [C.POINTER(VP), sz], "cuda_free": [VP],
            "cuda_copy_to_device_raw": [VP, VP, sz], "cuda_copy_from_device_raw": [VP, VP, sz],
            "cuda_copy_to_host": [VP, VP, sz, i],
            "cuda_create_conv_layer_weights_bf16": [C.POINTER(VP)] + [VP] * 8 + [i, i, i, f],
            "cuda_create_layer_weights_bf16_native": [C.POINTER(VP)] + [VP] * 11 + [i] * 5,
            "cuda_create_layer_workspace_bf16": [C.POINTER(VP), i, i, i, i, i],
            "cuda_create_conv_workspace": [C.POINTER(VP), i, i],
            "cuda_conv_state_reset": [VP, i, i, i],
            "cuda_paged_kvcache_create": [C.POINTER(VP), i, i, i, i],
            "cuda_create_decode_context": [C.POINTER(VP)] + [i] * 6 + [f, f, i, i],
            "cuda_set_decode_bf16_native": [VP, VP],
            "cuda_gather_embeddings": [VP, VP, VP, i, i],
            "cuda_prefill_batch": [VP, VP, VP, VP, VP, i],
            "cuda_decode_set_hidden": [VP, VP], "cuda_decode_set_hidden_from_gpu": [VP, VP],
            "cuda_decode_convert_fp16_to_bf16": [VP], "cuda_decode_step_gpu": [VP, i],
            "cuda_decode_step_batched": [VP] * 7 + [i],
            "cuda_rmsnorm": [VP, VP, VP, i, i, f], "cuda_gemm_fp16": [VP, VP, VP, i, i, i, C.c_bool, C.c_bool],
        }
        for name, args in sig.items():
            fn = getattr(L, name)
            fn.argtypes, fn.restype = args, i
        for name, args, res in (("cuda_set_decode_layer", [VP, i, i, VP, VP], None),
                                ("cuda_set_decode_paged_cache", [VP, VP, VP, i], None),
                                ("cuda_set_decode_paged_layer", [VP, i, VP], None),
                                ("cuda_set_decode_conv_workspace", [VP, VP], None),
                                ("cuda_decode_invalidate_graph", [VP], None),
                                ("cuda_conv_state_create", [i, i, i], VP),
                                ("cuda_decode_get_hidden_gpu_ptr", [VP], VP)):
            fn = getattr(L, name)
            fn.argtypes, fn.restype = args, res
        rt.cudaEventCreate.argtypes = [C.POINTER(VP)]
        rt.cudaEventRecord.argtypes = [VP, VP]
        rt.cudaEventSynchronize.argtypes = [VP]
        rt.cudaEventElapsedTime.argtypes = [C.POINTER(C.c_float), VP, VP]
        rt.cudaMemcpy.argtypes = [VP, VP, C.c_size_t, C.c_int]
        rt.cudaDeviceSynchronize.argtypes = []

    @staticmethod
    def _ok(rc, what):
        if rc != 0:
            raise Unavailable(f"the reference's {what} returned {rc}")

    def _alloc(self, nbytes: int) -> VP:
        p = VP()
        self._ok(self.lib.cuda_malloc(C.byref(p), nbytes), "cuda_malloc")
        return p

    def _upload(self, a: np.ndarray) -> VP:
        p = self._alloc(a.nbytes)
        self._ok(self.lib.cuda_copy_to_device_raw(p, _ptr(a), a.nbytes), "cuda_copy_to_device_raw")
        return p

    def _h2d(self, dst, a: np.ndarray):
        self._ok(self.lib.cuda_copy_to_device_raw(dst, _ptr(a), a.nbytes), "cuda_copy_to_device_raw")

    def sync(self):
        if self.rt.cudaDeviceSynchronize() != 0:
            raise Unavailable("cudaDeviceSynchronize reported an error after the reference's calls")

    def event(self) -> VP:
        e = VP()
        self.rt.cudaEventCreate(C.byref(e))
        return e

    def elapsed_ms(self, a, b) -> float:
        self.rt.cudaEventSynchronize(b)
        ms = C.c_float()
        self.rt.cudaEventElapsedTime(C.byref(ms), a, b)
        return float(ms.value)

    def _offset(self, p: VP, nbytes: int) -> VP:
        return VP(p.value + nbytes)

    # ------------------------------------------------------------------ conv states through the host
    def save_states(self, b: int):
        for i, st in self.conv_states.items():
            buf = self.saved[b].get(i)
            if buf is None:
                buf = self.saved[b][i] = np.empty(self.state_bytes, dtype=np.uint8)
            self._ok(self.lib.cuda_copy_from_device_raw(_ptr(buf), st, self.state_bytes), "copy_from_device_raw")

    def restore_states(self, b: int):
        for i, buf in self.saved[b].items():
            self._h2d(self.conv_states[i], buf)

    # ------------------------------------------------------------------ prefill (cuda_executor.go:307-419)
    def prefill(self, b: int, tokens) -> float:
        """Whole prompt of request ``b``; returns the device milliseconds of cuda_prefill_batch."""
        T, H, lib = len(tokens), self.H, self.lib
        if T >= MAX_CONTEXT:
            raise Unavailable("the reference's context is capped at 4,096 tokens")
        for st in self.conv_states.values():                    # batch_scheduler.go:222-227
            self._ok(lib.cuda_conv_state_reset(st, 1, H, self.K), "conv_state_reset")
        d_ids = self._upload(np.asarray(tokens, dtype=np.int32))
        d_pos = self._upload(np.arange(T, dtype=np.int32))
        d_slot = self._upload((self.tables[b][np.arange(T) // BLOCK] * BLOCK + np.arange(T) % BLOCK).astype(np.int32))
        d_emb, d_out = self._alloc(T * H * 2), self._alloc(H * 2)
        self._ok(lib.cuda_gather_embeddings(d_emb, self.embed, d_ids, H, T), "gather_embeddings")
        self._h2d(self.block_table_gpu, self.tables[b])
        e0, e1 = self.event(), self.event()
        self.rt.cudaEventRecord(e0, None)
        self._ok(lib.cuda_prefill_batch(self.ctx, d_emb, d_out, d_pos, d_slot, T), "cuda_prefill_batch")
        self.rt.cudaEventRecord(e1, None)
        ms = self.elapsed_ms(e0, e1)
        hidden = np.empty(H, dtype=np.float16)
        self._ok(lib.cuda_copy_from_device_raw(_ptr(hidden), d_out, H * 2), "copy_from_device_raw")
        for p in (d_ids, d_pos, d_slot, d_emb, d_out):
            lib.cuda_free(p)
        self.position[b] = T
        self.last_hidden[b] = hidden
        self.save_states(b)                                      # batch_scheduler.go:240-243
        return ms

    # ------------------------------------------------------------------ LM head (gpu_lmhead.go:141-290)
    def lm_head_device(self, hidden_gpu: VP):
        lib = self.lib
        self._ok(lib.cuda_rmsnorm(self.normed_gpu, hidden_gpu, self.final_norm, 1, self.H, self.eps), "cuda_rmsnorm")
        self._ok(lib.cuda_gemm_fp16(self.logits_gpu, self.normed_gpu, self.lm_head, 1, self.H, self.V, False, True),
                 "cuda_gemm_fp16")

    def logits_to_host(self) -> np.ndarray:
        self._ok(self.lib.cuda_copy_to_host(_ptr(self.logits_host), self.logits_gpu, self.V, 1), "cuda_copy_to_host")
        return self.logits_host

    def logits_to_host_argmax(self) -> int:
        return int(np.argmax(self.logits_to_host()))             # sampler.go:58-73

    def first_token(self, b: int) -> int:
        """batch_scheduler.go:489-502: the prefill's hidden state through the LM head."""
        self._ok(self.lib.cuda_decode_set_hidden(self.ctx, _ptr(self.last_hidden[b])), "decode_set_hidden")
        self._ok(self.lib.cuda_decode_convert_fp16_to_bf16(self.ctx), "convert_fp16_to_bf16")
        self._h2d(self.hidden_gpu, self.last_hidden[b])
        self.lm_head_device(self.hidden_gpu)
        return self.logits_to_host_argmax()

    # ------------------------------------------------------------------ decode, one request
    def decode_one(self, b: int, token: int, *, stock: bool) -> int:
        """One token of request ``b``.  ``stock``: everything batch_scheduler.go:421-557 does around
        the step (states through the host, graph invalidated, logits to the host, host argmax);
        else the device calls alone, the decode graph left alive, the token not read back."""
        lib = self.lib
        if self.position[b] + 1 >= MAX_CONTEXT:
            raise Unavailable("the reference's context is capped at 4,096 tokens")
        if stock:
            self.restore_states(b)
            lib.cuda_decode_invalidate_graph(self.ctx)
        self._ok(lib.cuda_decode_set_hidden_from_gpu(self.ctx, self._offset(self.embed, token * self.H * 2)),
                 "decode_set_hidden_from_gpu")
        self._ok(lib.cuda_decode_convert_fp16_to_bf16(self.ctx), "convert_fp16_to_bf16")
        if stock:
            self._h2d(self.block_table_gpu, self.tables[b])
        self._ok(lib.cuda_decode_step_gpu(self.ctx, self.position[b]), "cuda_decode_step_gpu")
        self.lm_head_device(VP(lib.cuda_decode_get_hidden_gpu_ptr(self.ctx)))
        self.position[b] += 1
        if not stock:
            return token
        nxt = self.logits_to_host_argmax()
        self.save_states(b)
        return nxt

    # ------------------------------------------------------------------ decode, N requests
    def decode_batched(self, tokens, *, stock: bool):
        """One token of requests 0..N-1 through cuda_decode_step_batched, as
        batch_scheduler.go:250-418 calls it: per-step device buffers, conv states of every request
        packed from and unpacked to their host copies, one LM head call and one logits copy per
        request.  Not ``stock``: the packed states stay on the device and logits are not read."""
        lib, N, H = self.lib, len(tokens), self.H
        if max(self.position[:N]) + 1 >= MAX_CONTEXT:
            raise Unavailable("the reference's context is capped at 4,096 tokens")
        d_emb = self._alloc(N * H * 2)
        for i, t in enumerate(tokens):                           # one device-to-device copy per request
            self.rt.cudaMemcpy(self._offset(d_emb, i * H * 2), self._offset(self.embed, int(t) * H * 2), H * 2, 3)
        pos = np.asarray(self.position[:N], dtype=np.int32)
        d_pos, d_len = self._upload(pos), self._upload(pos + 1)
        d_tab = self._upload(np.concatenate(self.tables[:N]))
        d_out = self._alloc(N * H * 2)
        if stock or getattr(self, "_packed", None) is None:
            packed = np.empty((self.n_conv, N, self.state_bytes), dtype=np.uint8)
            for ci, layer in enumerate(sorted(self.conv_states)):
                for b in range(N):
                    packed[ci, b] = self.saved[b][layer]
            d_states = self._upload(packed)
            if not stock:
                self._packed = d_states
        else:
            d_states = self._packed
        self._ok(lib.cuda_decode_step_batched(self.ctx, d_emb, d_out, d_pos, d_len, d_tab, d_states, N),
                 "cuda_decode_step_batched")
        out = list(tokens)
        for i in range(N):
            self.lm_head_device(self._offset(d_out, i * H * 2))
            if stock:
                out[i] = self.logits_to_host_argmax()
            self.position[i] += 1
        if stock:
            packed = np.empty((self.n_conv, N, self.state_bytes), dtype=np.uint8)
            self._ok(lib.cuda_copy_from_device_raw(_ptr(packed), d_states, packed.nbytes), "copy_from_device_raw")
            for ci, layer in enumerate(sorted(self.conv_states)):
                for b in range(N):
                    self.saved[b][layer] = packed[ci, b].copy()
            lib.cuda_free(d_states)
        for p in (d_emb, d_pos, d_len, d_tab, d_out):
            lib.cuda_free(p)
        return out


def _timed(ref: Reference, fn, steps: int):
    """(device ms per step, wall ms per step) of ``steps`` calls of ``fn`` in one region."""
    a, b = ref.event(), ref.event()
    ref.sync()
    t0 = time.perf_counter()
    ref.rt.cudaEventRecord(a, None)
    for _ in range(steps):
        fn()
    ref.rt.cudaEventRecord(b, None)
    dev = ref.elapsed_ms(a, b)
    ref.sync()
    return dev / steps, (time.perf_counter() - t0) * 1e3 / steps


def run(cfg: dict, *, batch: int, steps: int, warmup: int, prompt_len: int, seed: int = 0) -> dict:
    """Prefill ``batch`` requests of ``prompt_len`` tokens, then time decode at batch 1 and at
    ``batch``.  Returns the measurements; raises :class:`Unavailable` with the reason otherwise."""
    rng = np.random.default_rng(seed + 1)
    ref = Reference(cfg, max_batch=batch, seed=seed)
    V = cfg["vocab_size"]
    room = MAX_CONTEXT - prompt_len - 8
    per_region = 2 * (warmup + steps)                            # the kernel-only and the stock region
    if per_region * (2 if batch > 1 else 1) > room:
        raise Unavailable(f"{steps} steps after a {prompt_len}-token prompt pass the reference's 4,096-token context")
    prefill_ms = []
    for b in range(batch):
        prefill_ms.append(ref.prefill(b, rng.integers(0, V, prompt_len).tolist()))
    out = {"prefill_ms": prefill_ms[-1] if len(prefill_ms) > 1 else prefill_ms[0], "prefill_first_ms": prefill_ms[0],
           "prefill_tokens": prompt_len, "launch_note": "298-302 graph nodes per token (reference CHANGELOG.md:136,164)"}
    # ---- one request (request 0): first token from the prefill's hidden state, then decode
    ref.restore_states(0)
    ref._h2d(ref.block_table_gpu, ref.tables[0])
    tok = [ref.first_token(0)]

    def one_kernel():
        ref.decode_one(0, tok[0], stock=False)

    def one_stock():
        tok[0] = ref.decode_one(0, tok[0], stock=True)

    for _ in range(warmup):
        one_kernel()
    out["b1_kernel_ms"], _ = _timed(ref, one_kernel, steps)
    ref.save_states(0)
    for _ in range(warmup):
        one_stock()
    _, out["b1_stock_ms"] = _timed(ref, one_stock, steps)
    # ---- `batch` requests through the batched entry
    if batch > 1:
        toks = [rng.integers(0, V, batch).tolist()]

        def n_kernel():
            ref.decode_batched(toks[0], stock=False)

        def n_stock():
            toks[0] = ref.decode_batched(toks[0], stock=True)

        for _ in range(warmup):
            n_stock()
        _, out["bN_stock_ms"] = _timed(ref, n_stock, steps)
        for _ in range(warmup):
            n_kernel()
        out["bN_kernel_ms"], _ = _timed(ref, n_kernel, steps)
    ref.sync()
    out["h2d_bytes_per_step"] = 4 * batch * (2 + MAX_BLOCKS) + ref.n_conv * batch * ref.state_bytes
    out["d2h_bytes_per_step"] = 4 * ref.V * batch + ref.n_conv * batch * ref.state_bytes
    return out

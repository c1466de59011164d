"""OpenAI-compatible server bindings (C++ front end in ``csrc/server``) and the glue that lets a Python engine act as
its backend.  ``Server.handle`` runs a request in process (tests, embedding); ``Server.start`` listens on a socket."""
from __future__ import annotations

import ctypes as C
import json
from typing import Callable, List, Optional, Sequence

from .. import _lib

_GEN_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_longlong, C.POINTER(C.c_int), C.c_int, C.c_char_p, C.c_char_p)


def _h():
    h = _lib.host_lib()
    if not getattr(h, "_srv_sig", False):
        vp, i, cp = C.c_void_p, C.c_int, C.c_char_p
        ip = C.POINTER(C.c_int)
        sig = {
            "b2h_server_new": ([cp, cp, i], vp), "b2h_server_free": ([vp], None),
            "b2h_server_use_mock": ([vp, ip, i, i, i], None), "b2h_server_mock_calls": ([vp], vp),
            "b2h_server_use_callback": ([vp, _GEN_FN, vp, i], None), "b2h_server_set_images": ([vp, i], i),
            "b2h_server_set_metrics": ([vp, C.c_char_p], None),
            "b2h_stream_push": ([vp, C.c_longlong, ip, i, i, cp], i), "b2h_stream_cancelled": ([vp, C.c_longlong], i),
            "b2h_server_handle": ([vp, cp, cp, cp, cp, ip], vp),
            "b2h_server_start": ([vp, cp, i], i), "b2h_server_stop": ([vp], None),
            "b2h_tok_new": ([cp, cp, i], vp), "b2h_tok_free": ([vp], None), "b2h_tok_encode": ([vp, cp, ip, i], i),
            "b2h_tok_decode": ([vp, ip, i, i], vp), "b2h_detok_new": ([vp, i], vp), "b2h_detok_free": ([vp], None),
            "b2h_detok_push": ([vp, ip, i], vp), "b2h_detok_finish": ([vp], vp),
            "b2h_render_chat": ([cp, cp, i, i, i], vp), "b2h_parse_output": ([cp, cp, i, i], vp),
            "b2h_free_str": ([vp], None), "b2h_render_template": ([cp, cp, cp, i], vp),
        }
        for name, (args, res) in sig.items():
            fn = getattr(h, name)
            fn.argtypes, fn.restype = args, res
        h._srv_sig = True
    return h


def _take(p) -> str:
    s = C.cast(p, C.c_char_p).value.decode("utf-8", errors="replace")
    _h().b2h_free_str(p)
    return s


def _ints(xs: Sequence[int]):
    return (C.c_int * len(xs))(*xs)


class Tokenizer:
    def __init__(self, tokenizer_json_text: str):
        err = C.create_string_buffer(256)
        self._t = _h().b2h_tok_new(tokenizer_json_text.encode(), err, 256)
        if not self._t:
            raise ValueError(err.value.decode())

    def __del__(self):
        if getattr(self, "_t", None):
            _h().b2h_tok_free(self._t)

    def encode(self, text: str) -> List[int]:
        cap = 4 * len(text.encode()) + 16
        buf = (C.c_int * cap)()
        n = _h().b2h_tok_encode(self._t, text.encode(), buf, cap)
        return list(buf[:n])

    def decode(self, ids: Sequence[int], skip_special: bool = True) -> str:
        return _take(_h().b2h_tok_decode(self._t, _ints(ids), len(ids), 1 if skip_special else 0))

    def stream_decode(self, ids: Sequence[int], step: int = 1, skip_special: bool = True) -> List[str]:
        d = _h().b2h_detok_new(self._t, 1 if skip_special else 0)
        out = []
        for i in range(0, len(ids), step):
            chunk = list(ids[i:i + step])
            out.append(_take(_h().b2h_detok_push(d, _ints(chunk), len(chunk))))
        out.append(_take(_h().b2h_detok_finish(d)))
        _h().b2h_detok_free(d)
        return out


def render_chat(messages: list, tools: Optional[list] = None, add_generation_prompt: bool = True,
                enable_thinking: bool = True, continue_final: bool = False) -> str:
    return _take(_h().b2h_render_chat(json.dumps(messages).encode(), json.dumps(tools or []).encode(),
                                      int(add_generation_prompt), int(enable_thinking), int(continue_final)))


def render_template(source: str, **context) -> str:
    """Renders a Jinja chat template (the subset that chat templates use) with ``context`` as its variables."""
    err = C.create_string_buffer(512)
    p = _h().b2h_render_template(source.encode(), json.dumps(context).encode(), err, 512)
    if not p:
        raise ValueError(err.value.decode(errors="replace"))
    return _take(p)


def parse_output(text: str, tools: Optional[list] = None, starts_in_reasoning: bool = False, chunk: int = 0) -> dict:
    return json.loads(_take(_h().b2h_parse_output(text.encode(), json.dumps(tools or []).encode(), int(starts_in_reasoning), chunk)))


class Server:
    def __init__(self, tokenizer_json: str, model_name: str = "b200-engine", generation_config: Optional[dict] = None,
                 eos_token_ids: Sequence[int] = (), max_tokens_default: int = 32768, chat_template: str = "",
                 bos_token: str = "", eos_token: str = ""):
        """``chat_template``: Jinja source (``tokenizer_config.json``); empty selects the built-in ChatML renderer."""
        cfg = {"tokenizer_json": tokenizer_json, "model_name": model_name, "generation_config": generation_config or {},
               "eos_token_ids": list(eos_token_ids), "max_tokens_default": max_tokens_default, "chat_template": chat_template,
               "bos_token": bos_token, "eos_token": eos_token}
        err = C.create_string_buffer(256)
        self._s = _h().b2h_server_new(json.dumps(cfg).encode(), err, 256)
        if not self._s:
            raise ValueError(err.value.decode())
        self._cb = None

    def use_mock(self, script: Sequence[int], step: int = 1, supports_images: bool = False):
        _h().b2h_server_use_mock(self._s, _ints(script), len(script), step, int(supports_images))

    def mock_calls(self) -> list:
        return json.loads(_take(_h().b2h_server_mock_calls(self._s)))

    def use_engine(self, generate: Callable[[int, List[int], dict, str], None], context_length: int = 262144,
                   supports_images: bool = False):
        """``generate(req_id, prompt_ids, sampling, session_id)`` must return at once; the engine later calls
        :meth:`push` with each step's tokens.  With ``supports_images`` chat requests may carry ``image_url`` parts
        (base64 ``data:`` URLs); they arrive as ``sampling["images"]``, one per ``<|image_pad|>`` token of the prompt."""
        def tramp(_user, req_id, prompt, n, sampling, session):
            generate(req_id, [prompt[i] for i in range(n)], json.loads(sampling.decode()), session.decode())
        self._cb = _GEN_FN(tramp)
        _h().b2h_server_use_callback(self._s, self._cb, None, context_length)
        _h().b2h_server_set_images(self._s, int(supports_images))

    def set_metrics(self, text: str):
        """Engine-side gauges shown by ``/metrics`` after the request counters (Prometheus text format)."""
        _h().b2h_server_set_metrics(self._s, text.encode())

    def push(self, req_id: int, ids: Sequence[int], finished: bool = False, error: Optional[str] = None) -> bool:
        """Returns True when the client is gone (stop generating)."""
        r = _h().b2h_stream_push(self._s, req_id, _ints(ids), len(ids), int(finished), error.encode() if error else None)
        return r != 0

    def cancelled(self, req_id: int) -> bool:
        return bool(_h().b2h_stream_cancelled(self._s, req_id))

    def handle(self, method: str, path: str, body: Optional[dict] = None, session_id: str = ""):
        st = C.c_int()
        text = _take(_h().b2h_server_handle(self._s, method.encode(), path.encode(), session_id.encode(),
                                            json.dumps(body).encode() if body is not None else b"", C.byref(st)))
        return st.value, text

    def start(self, host: str = "127.0.0.1", port: int = 0) -> int:
        p = _h().b2h_server_start(self._s, host.encode(), port)
        if p < 0:
            raise OSError("cannot listen")
        return p

    def stop(self):
        _h().b2h_server_stop(self._s)

    def __del__(self):
        if getattr(self, "_s", None):
            try:
                self.stop()
            finally:
                _h().b2h_server_free(self._s)
                self._s = None

"""gRPC front end of the serving loop: a streaming `Decode` and a `HealthCheck`, the two calls of the orchestrator service that
the reference serves through JetStream (src/maxtext/inference/maxengine/maxengine_server.py:64-105).

  service jetstream_proto.Orchestrator
    rpc Decode(DecodeRequest) returns (stream DecodeResponse)
    rpc HealthCheck(HealthCheckRequest) returns (HealthCheckResponse)

Messages are protobuf on the wire, encoded and decoded here by hand (no generated code; `protoc` is not part of this
environment). The layout is modelled on JetStream's published proto:

  DecodeRequest   { max_tokens = 4 (int32); text_content = 5 { text = 1 }; token_content = 6 { token_ids = 1 (packed int32) } }
  DecodeResponse  { stream_content = 3 { samples = 1 { text = 1; token_ids = 2 (packed int32) } } }
  HealthCheckResponse { is_live = 1 (bool) }

Tokens are streamed as they are generated: one DecodeResponse per poll of the request's output while the continuous-batching
loop advances it, then the stream ends.
"""
from __future__ import annotations

import sys
import time
from concurrent import futures

from ..input_pipeline.record_formats import _enc_varint, _fields, _ld, _varint

SERVICE = "jetstream_proto.Orchestrator"


# ------------------------------------------------------------------------------------------------- messages
def _packed_ints(buf) -> list[int]:
  out, i = [], 0
  while i < len(buf):
    v, i = _varint(buf, i)
    out.append(v - (1 << 64) if v >> 63 else v)
  return out


def decode_request(payload: bytes) -> dict:
  req = {"max_tokens": 0, "text": None, "token_ids": None}
  for num, wt, v in _fields(memoryview(payload)):
    if num == 4 and wt == 0:
      req["max_tokens"] = int(v)
    elif num == 5 and wt == 2:
      for n2, _, x in _fields(v):
        if n2 == 1:
          req["text"] = bytes(x).decode("utf-8")
    elif num == 6 and wt == 2:
      ids = []
      for n2, w2, x in _fields(v):
        if n2 == 1:
          ids.extend(_packed_ints(x) if w2 == 2 else [int(x)])
      req["token_ids"] = ids
  return req


def encode_request(text: str | None = None, token_ids=None, max_tokens: int = 32) -> bytes:
  out = _enc_varint((4 << 3) | 0) + _enc_varint(int(max_tokens))
  if token_ids is not None:
    out += _ld(6, _ld(1, b"".join(_enc_varint(int(t)) for t in token_ids)))
  else:
    out += _ld(5, _ld(1, (text or "").encode("utf-8")))
  return out


def encode_response(text: str, token_ids) -> bytes:
  sample = _ld(1, text.encode("utf-8")) + _ld(2, b"".join(_enc_varint(int(t)) for t in token_ids))
  return _ld(3, _ld(1, sample))


def decode_response(payload: bytes) -> dict:
  out = {"text": "", "token_ids": []}
  for num, _, v in _fields(memoryview(payload)):
    if num != 3:
      continue
    for n2, _, sample in _fields(v):
      if n2 != 1:
        continue
      for n3, w3, x in _fields(sample):
        if n3 == 1:
          out["text"] = bytes(x).decode("utf-8")
        elif n3 == 2:
          out["token_ids"].extend(_packed_ints(x) if w3 == 2 else [int(x)])
  return out


# ------------------------------------------------------------------------------------------------- service
def _handlers(loop):
  import grpc
  cfg, tok = loop.config, loop.tok

  def decode(request: bytes, context):
    req = decode_request(request)
    toks = req["token_ids"] if req["token_ids"] is not None else tok.encode(req["text"] or "", add_bos=bool(cfg.add_bos))
    toks = [int(t) for t in toks][-int(cfg.max_prefill_predict_length):] or [0]
    max_new = max(1, min(int(req["max_tokens"] or 32), int(cfg.max_target_length) - len(toks) - 1))
    item = loop.submit(toks, max_new)
    sent = 0
    deadline = time.monotonic() + 600.0
    while time.monotonic() < deadline and context.is_active():
      r = item["request"]
      out = list(r.output) if r is not None else []
      if len(out) > sent:
        new = out[sent:]
        sent = len(out)
        yield encode_response(tok.decode(new), new)
      if item["event"].is_set() and sent >= len(item["request"].output):
        return
      time.sleep(0.002)
    context.abort(grpc.StatusCode.DEADLINE_EXCEEDED, "generation timed out")

  def health(request: bytes, context):
    return _enc_varint((1 << 3) | 0) + _enc_varint(1)

  ident = lambda b: b  # noqa: E731
  return grpc.method_handlers_generic_handler(SERVICE, {
      "Decode": grpc.unary_stream_rpc_method_handler(decode, request_deserializer=ident, response_serializer=ident),
      "HealthCheck": grpc.unary_unary_rpc_method_handler(health, request_deserializer=ident, response_serializer=ident),
  })


def serve(loop, port: int = 9000, workers: int = 16):
  """Starts the server on 127.0.0.1:`port` (0 = any free port); returns (server, bound port)."""
  import grpc
  server = grpc.server(futures.ThreadPoolExecutor(max_workers=workers))
  server.add_generic_rpc_handlers((_handlers(loop),))
  bound = server.add_insecure_port(f"127.0.0.1:{int(port)}")
  server.start()
  return server, bound


class Client:
  """Minimal client of the two calls (tests, smoke checks)."""

  def __init__(self, address: str):
    import grpc
    self.channel = grpc.insecure_channel(address)
    ident = lambda b: b  # noqa: E731
    self._decode = self.channel.unary_stream(f"/{SERVICE}/Decode", request_serializer=ident, response_deserializer=ident)
    self._health = self.channel.unary_unary(f"/{SERVICE}/HealthCheck", request_serializer=ident, response_deserializer=ident)

  def decode(self, text=None, token_ids=None, max_tokens=32):
    for chunk in self._decode(encode_request(text, token_ids, max_tokens)):
      yield decode_response(chunk)

  def healthy(self) -> bool:
    return any(num == 1 and int(v) == 1 for num, _, v in _fields(memoryview(self._health(b""))))

  def close(self):
    self.channel.close()


def main(argv=None):
  from ..config import pyconfig
  from .maxengine_server import ServingLoop
  argv = list(sys.argv if argv is None else argv)
  port = next((int(a.split("=", 1)[1]) for a in argv if a.startswith("port=")), 9000)
  argv = [a for a in argv if not a.startswith("port=")]
  loop = ServingLoop(pyconfig.initialize(argv)).start()
  server, bound = serve(loop, port)
  print(f"serving {SERVICE} on 127.0.0.1:{bound}", flush=True)
  server.wait_for_termination()


if __name__ == "__main__":
  main()

"""gRPC transport of the parameter server, wire-compatible with the reference's ``xmhps.ParameterService``.

The reference serves its CachePS over gRPC (src/grpc_ps/proto/ps.proto, src/grpc_ps/grpc_ps_server.cpp:36-118) and
its client cuts a request into sub-requests of ``MAX_PARAMETER_BATCH`` keys issued concurrently
(src/grpc_ps/grpc_ps_client.cpp:52-140).  This module puts the same service in front of the native shard
(``ParameterServer``: the KV engines and the server-side optimizer of ``csrc/runtime/ps.cpp``):

* service ``/xmhps.ParameterService/{GetParameter, PutParameter, Command}`` with the reference's messages.  The
  message classes are built from a descriptor written here (no generated ``_pb2`` files, no ``protoc``); field
  numbers and types are those of ps.proto, so a stock reference client can talk to this server and this client to a
  stock reference server.
* ``GetParameterRequest.keys`` is the raw little-endian ``uint64`` key array, ``parameter_value`` is the packed record
  block ``[int32 n][int32 end_offset[n]]{u64 key; int32 dim; float emb[dim]}`` (``ps.client.pack_records``); an absent
  key comes back as a record of dim 0.
* ``Command``: CLEAR_PS, RELOAD_PS (arg2 = checkpoint files) and LOAD_FAKE_DATA (arg1[0] = int64 count) as in the
  reference; two commands beyond it, SAVE_PS (arg1[0] = path) and STATS.
* one method beyond the reference, ``UpdateParameter`` (a ``PutParameterRequest`` whose records are gradients, applied
  by the server-side optimizer), because the reference's trainers update through Put of client-computed rows while the
  native shard owns the optimizer state.

* the standard health-check service ``/grpc.health.v1.Health/Check`` (the reference enables gRPC's default one,
  grpc_ps_server.cpp:131): SERVING while the shard answers, for the service names "" and "xmhps.ParameterService".

* server reflection ``/grpc.reflection.v1alpha.ServerReflection/ServerReflectionInfo`` (and the same under ``v1``), which
  the reference switches on beside the health service (grpc_ps_server.cpp:131-146): ``list_services``,
  ``file_containing_symbol`` and ``file_by_filename`` answer with the descriptor written here, so generic tools can
  list the service and call it without a ``.proto`` file.

``GrpcParameterClient`` has the API of ``ps.client.ParameterClient`` and can be handed to
``AllShardsParameterClient``.
"""
from __future__ import annotations

import struct
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional, Tuple

import grpc
import numpy as np
import torch
from google.protobuf import descriptor_pb2, descriptor_pool, message_factory

from .client import MAX_PARAMETER_BATCH, ParameterServer, _keys, pack_records, unpack_records

SERVICE = "xmhps.ParameterService"
CLEAR_PS, RELOAD_PS, LOAD_FAKE_DATA, SAVE_PS, STATS = 0, 1, 2, 3, 4


def _build_messages():
    f = descriptor_pb2.FileDescriptorProto()
    f.name = "recstore_b200/ps.proto"
    f.package = "xmhps"
    f.syntax = "proto3"
    T = descriptor_pb2.FieldDescriptorProto

    def msg(name, fields):
        m = f.message_type.add()
        m.name = name
        for fname, num, ftype, label, tname in fields:
            fd = m.field.add()
            fd.name, fd.number, fd.type, fd.label = fname, num, ftype, label
            if tname:
                fd.type_name = tname
    e = f.enum_type.add()
    e.name = "PSCommand"
    for n, v in (("CLEAR_PS", 0), ("RELOAD_PS", 1), ("LOAD_FAKE_DATA", 2), ("SAVE_PS", 3), ("STATS", 4)):
        ev = e.value.add()
        ev.name, ev.number = n, v
    opt, rep = T.LABEL_OPTIONAL, T.LABEL_REPEATED
    msg("GetParameterRequest", [("keys", 1, T.TYPE_BYTES, opt, ""), ("model_name", 2, T.TYPE_BYTES, opt, ""),
                                ("perf", 3, T.TYPE_BOOL, opt, "")])
    msg("GetParameterResponse", [("parameter_value", 1, T.TYPE_BYTES, opt, ""), ("keys", 2, T.TYPE_BYTES, opt, "")])
    msg("CommandRequest", [("command", 1, T.TYPE_ENUM, opt, ".xmhps.PSCommand"), ("arg1", 2, T.TYPE_BYTES, rep, ""),
                           ("arg2", 3, T.TYPE_BYTES, rep, ""), ("arg3", 4, T.TYPE_BYTES, rep, "")])
    msg("CommandResponse", [("reply", 1, T.TYPE_STRING, opt, "")])
    msg("PutParameterRequest", [("parameter_value", 2, T.TYPE_BYTES, opt, "")])
    msg("PutParameterResponse", [("sucess", 1, T.TYPE_BOOL, opt, "")])
    svc = f.service.add()
    svc.name = "ParameterService"
    for name, req, resp in (("GetParameter", "GetParameterRequest", "GetParameterResponse"),
                            ("Command", "CommandRequest", "CommandResponse"),
                            ("PutParameter", "PutParameterRequest", "PutParameterResponse"),
                            ("UpdateParameter", "PutParameterRequest", "PutParameterResponse")):
        m = svc.method.add()
        m.name, m.input_type, m.output_type = name, ".xmhps." + req, ".xmhps." + resp
    pool = descriptor_pool.DescriptorPool()
    pool.Add(f)
    out = {n: message_factory.GetMessageClass(pool.FindMessageTypeByName("xmhps." + n))
           for n in ("GetParameterRequest", "GetParameterResponse", "CommandRequest", "CommandResponse",
                     "PutParameterRequest", "PutParameterResponse")}
    out["__file__"] = f
    return out


def _build_reflection_messages():
    """grpc.reflection.v1alpha (reflection.proto): the request / response pair of ServerReflectionInfo and their parts."""
    f = descriptor_pb2.FileDescriptorProto()
    f.name = "recstore_b200/reflection.proto"
    f.package = "grpc.reflection.v1alpha"
    f.syntax = "proto3"
    T = descriptor_pb2.FieldDescriptorProto
    opt, rep = T.LABEL_OPTIONAL, T.LABEL_REPEATED
    P = ".grpc.reflection.v1alpha."

    def msg(name, fields, oneof=None):
        m = f.message_type.add()
        m.name = name
        if oneof:
            m.oneof_decl.add().name = oneof
        for fname, num, ftype, label, tname, in_oneof in fields:
            fd = m.field.add()
            fd.name, fd.number, fd.type, fd.label = fname, num, ftype, label
            if tname:
                fd.type_name = tname
            if in_oneof:
                fd.oneof_index = 0
    msg("ExtensionRequest", [("containing_type", 1, T.TYPE_STRING, opt, "", False), ("extension_number", 2, T.TYPE_INT32, opt, "", False)])
    msg("ServerReflectionRequest", [("host", 1, T.TYPE_STRING, opt, "", False),
                                    ("file_by_filename", 3, T.TYPE_STRING, opt, "", True),
                                    ("file_containing_symbol", 4, T.TYPE_STRING, opt, "", True),
                                    ("file_containing_extension", 5, T.TYPE_MESSAGE, opt, P + "ExtensionRequest", True),
                                    ("all_extension_numbers_of_type", 6, T.TYPE_STRING, opt, "", True),
                                    ("list_services", 7, T.TYPE_STRING, opt, "", True)], oneof="message_request")
    msg("FileDescriptorResponse", [("file_descriptor_proto", 1, T.TYPE_BYTES, rep, "", False)])
    msg("ExtensionNumberResponse", [("base_type_name", 1, T.TYPE_STRING, opt, "", False), ("extension_number", 2, T.TYPE_INT32, rep, "", False)])
    msg("ServiceResponse", [("name", 1, T.TYPE_STRING, opt, "", False)])
    msg("ListServiceResponse", [("service", 1, T.TYPE_MESSAGE, rep, P + "ServiceResponse", False)])
    msg("ErrorResponse", [("error_code", 1, T.TYPE_INT32, opt, "", False), ("error_message", 2, T.TYPE_STRING, opt, "", False)])
    msg("ServerReflectionResponse", [("valid_host", 1, T.TYPE_STRING, opt, "", False),
                                     ("original_request", 2, T.TYPE_MESSAGE, opt, P + "ServerReflectionRequest", False),
                                     ("file_descriptor_response", 4, T.TYPE_MESSAGE, opt, P + "FileDescriptorResponse", True),
                                     ("all_extension_numbers_response", 5, T.TYPE_MESSAGE, opt, P + "ExtensionNumberResponse", True),
                                     ("list_services_response", 6, T.TYPE_MESSAGE, opt, P + "ListServiceResponse", True),
                                     ("error_response", 7, T.TYPE_MESSAGE, opt, P + "ErrorResponse", True)], oneof="message_response")
    pool = descriptor_pool.DescriptorPool()
    pool.Add(f)
    return {n: message_factory.GetMessageClass(pool.FindMessageTypeByName("grpc.reflection.v1alpha." + n))
            for n in ("ServerReflectionRequest", "ServerReflectionResponse")}


_M = _build_messages()
_PS_FILE = _M.pop("__file__")
_R = _build_reflection_messages()
ServerReflectionRequest, ServerReflectionResponse = _R["ServerReflectionRequest"], _R["ServerReflectionResponse"]
REFLECTION_SERVICES = ("grpc.reflection.v1alpha.ServerReflection", "grpc.reflection.v1.ServerReflection")
GetParameterRequest, GetParameterResponse = _M["GetParameterRequest"], _M["GetParameterResponse"]
CommandRequest, CommandResponse = _M["CommandRequest"], _M["CommandResponse"]
PutParameterRequest, PutParameterResponse = _M["PutParameterRequest"], _M["PutParameterResponse"]

_CHANNEL_OPTIONS = [("grpc.max_send_message_length", 256 << 20), ("grpc.max_receive_message_length", 256 << 20)]


class GrpcParameterServer:
    """Serves one ``ParameterServer`` shard on ``host:port`` (``port=0`` picks a free port; see ``.port``)."""

    def __init__(self, ps: ParameterServer, port: int = 0, host: str = "127.0.0.1", workers: int = 8):
        self.ps = ps
        self.requests = 0
        self.keys_served = 0
        self._server = grpc.server(ThreadPoolExecutor(max_workers=workers), options=_CHANNEL_OPTIONS)
        un = grpc.unary_unary_rpc_method_handler
        handlers = {
            "GetParameter": un(self._get, GetParameterRequest.FromString, GetParameterResponse.SerializeToString),
            "PutParameter": un(self._put, PutParameterRequest.FromString, PutParameterResponse.SerializeToString),
            "UpdateParameter": un(self._update, PutParameterRequest.FromString, PutParameterResponse.SerializeToString),
            "Command": un(self._command, CommandRequest.FromString, CommandResponse.SerializeToString),
        }
        health = {"Check": un(self._health, lambda b: b, lambda b: b)}
        reflect = {"ServerReflectionInfo": grpc.stream_stream_rpc_method_handler(
            self._reflect, ServerReflectionRequest.FromString, ServerReflectionResponse.SerializeToString)}
        self._server.add_generic_rpc_handlers(
            (grpc.method_handlers_generic_handler(SERVICE, handlers),
             grpc.method_handlers_generic_handler("grpc.health.v1.Health", health))
            + tuple(grpc.method_handlers_generic_handler(name, reflect) for name in REFLECTION_SERVICES))
        self.port = self._server.add_insecure_port(f"{host}:{int(port)}")
        if self.port == 0:
            raise OSError(f"cannot bind {host}:{port}")
        self._server.start()

    # handlers ---------------------------------------------------------------------------
    def _health(self, raw: bytes, ctx):
        """grpc.health.v1: HealthCheckRequest{string service = 1} -> HealthCheckResponse{ServingStatus status = 1}; the two
        messages are small enough to be read and written as raw protobuf bytes."""
        service = b""
        if raw:
            if raw[0] != 0x0a or len(raw) < 2 or raw[1] != len(raw) - 2:
                ctx.abort(grpc.StatusCode.INVALID_ARGUMENT, "malformed HealthCheckRequest")
            service = raw[2:]
        if service not in (b"", SERVICE.encode()):
            ctx.abort(grpc.StatusCode.NOT_FOUND, "unknown service")
        try:
            len(self.ps)                      # the shard still answers
            return b"\x08\x01"                # SERVING
        except Exception:
            return b"\x08\x02"                # NOT_SERVING

    def _reflect(self, requests, ctx):
        """One answer per request of the stream.  Symbols of the parameter service resolve to the descriptor this module
        built; the health and reflection services are listed but carry no descriptor here."""
        symbols = {SERVICE} | {f"xmhps.{m.name}" for m in _PS_FILE.message_type} | {f"xmhps.{e.name}" for e in _PS_FILE.enum_type} \
            | {f"{SERVICE}.{m.name}" for m in _PS_FILE.service[0].method}
        for req in requests:
            rep = ServerReflectionResponse(valid_host=req.host, original_request=req)
            which = req.WhichOneof("message_request")
            if which == "list_services":
                for name in (SERVICE, "grpc.health.v1.Health") + REFLECTION_SERVICES:
                    rep.list_services_response.service.add().name = name
            elif which == "file_containing_symbol" and req.file_containing_symbol in symbols:
                rep.file_descriptor_response.file_descriptor_proto.append(_PS_FILE.SerializeToString())
            elif which == "file_by_filename" and req.file_by_filename == _PS_FILE.name:
                rep.file_descriptor_response.file_descriptor_proto.append(_PS_FILE.SerializeToString())
            elif which == "all_extension_numbers_of_type" and req.all_extension_numbers_of_type in symbols:
                rep.all_extension_numbers_response.base_type_name = req.all_extension_numbers_of_type     # proto3: none
            elif which is None:
                rep.error_response.error_code = grpc.StatusCode.INVALID_ARGUMENT.value[0]
                rep.error_response.error_message = "empty reflection request"
            else:
                rep.error_response.error_code = grpc.StatusCode.NOT_FOUND.value[0]
                rep.error_response.error_message = f"{which}: not known to this server"
            yield rep

    def _get(self, req, ctx):
        raw = req.keys
        if len(raw) % 8:
            ctx.abort(grpc.StatusCode.INVALID_ARGUMENT, "keys must be a uint64 array")
        keys = torch.from_numpy(np.frombuffer(raw, dtype=np.int64).copy())
        rows, found = self.ps.GetParameterWithMask(keys)
        self.requests += 1
        self.keys_served += keys.numel()
        dims = torch.where(found, self.ps.dim, 0).to(torch.int32)
        return GetParameterResponse(parameter_value=pack_records(keys, rows, dims))

    def _records(self, req, ctx):
        try:
            k, d, v = unpack_records(req.parameter_value, self.ps.dim)
        except Exception as e:                                     # malformed block: refuse the call, keep serving
            ctx.abort(grpc.StatusCode.INVALID_ARGUMENT, str(e))
        ok = d == self.ps.dim
        return k[ok], v[ok]

    def _put(self, req, ctx):
        k, v = self._records(req, ctx)
        self.ps.PutParameter(k, v)
        self.requests += 1
        return PutParameterResponse(sucess=True)

    def _update(self, req, ctx):
        k, g = self._records(req, ctx)
        self.ps.UpdateParameter(k, g)
        self.requests += 1
        return PutParameterResponse(sucess=True)

    def _command(self, req, ctx):
        self.requests += 1
        c = req.command
        if c == CLEAR_PS:
            self.ps.ClearPS()
            return CommandResponse(reply="cleared")
        if c == LOAD_FAKE_DATA:
            if len(req.arg1) != 1 or len(req.arg1[0]) != 8:
                ctx.abort(grpc.StatusCode.INVALID_ARGUMENT, "LOAD_FAKE_DATA wants arg1 = [int64]")
            n = struct.unpack("<q", req.arg1[0])[0]
            self.ps.LoadFakeData(n)
            return CommandResponse(reply=str(n))
        if c == RELOAD_PS:
            files = [a.decode() for a in req.arg2] or [a.decode() for a in req.arg1]
            if not files:
                ctx.abort(grpc.StatusCode.INVALID_ARGUMENT, "RELOAD_PS wants checkpoint paths")
            try:
                for p in files:
                    self.ps.LoadCkpt(p)
            except Exception as e:
                ctx.abort(grpc.StatusCode.NOT_FOUND, str(e))
            return CommandResponse(reply=str(len(self.ps)))
        if c == SAVE_PS:
            try:
                self.ps.SaveCkpt(req.arg1[0].decode())
            except Exception as e:
                ctx.abort(grpc.StatusCode.FAILED_PRECONDITION, str(e))
            return CommandResponse(reply="saved")
        if c == STATS:
            return CommandResponse(reply=f"{len(self.ps)} {self.requests} {self.keys_served}")
        ctx.abort(grpc.StatusCode.INVALID_ARGUMENT, f"unknown command {c}")

    def stop(self, grace: Optional[float] = 0.5) -> None:
        if self._server is not None:
            self._server.stop(grace).wait()
            self._server = None

    close = stop

    def __del__(self):
        try:
            self.stop(0)
        except Exception:
            pass


class GrpcParameterClient:
    """Client of one shard over gRPC; same verbs as ``ps.client.ParameterClient``.  ``timeout_s`` bounds every call, a
    server that is gone raises ``grpc.RpcError`` instead of hanging the trainer."""

    def __init__(self, host: str, port: int, shard: int = 0, emb_dim: int = 32, timeout_s: float = 30.0):
        self._channel = grpc.insecure_channel(f"{host}:{int(port)}", options=_CHANNEL_OPTIONS)
        self._shard, self.dim, self.timeout_s = shard, emb_dim, timeout_s

        def stub(name, req, resp):
            return self._channel.unary_unary(f"/{SERVICE}/{name}", request_serializer=req.SerializeToString,
                                             response_deserializer=resp.FromString)
        self._get = stub("GetParameter", GetParameterRequest, GetParameterResponse)
        self._put = stub("PutParameter", PutParameterRequest, PutParameterResponse)
        self._upd = stub("UpdateParameter", PutParameterRequest, PutParameterResponse)
        self._cmd = stub("Command", CommandRequest, CommandResponse)
        self._rpcs = {}
        self._next_rpc = 0

    def shard(self) -> int:
        return self._shard

    # Get: sub-requests in flight together, reassembled in request order -----------------------
    def _issue_get(self, k: torch.Tensor, perf: bool):
        a = k.numpy()
        return [self._get.future(GetParameterRequest(keys=a[s:s + MAX_PARAMETER_BATCH].tobytes(), perf=perf),
                                 timeout=self.timeout_s) for s in range(0, len(a), MAX_PARAMETER_BATCH)]

    def _collect_get(self, futs, n: int) -> Tuple[torch.Tensor, torch.Tensor]:
        out = torch.zeros(n, self.dim)
        found = torch.zeros(n, dtype=torch.bool)
        at = 0
        for f in futs:
            _, d, v = unpack_records(f.result().parameter_value, self.dim)
            out[at:at + v.shape[0]] = v
            found[at:at + v.shape[0]] = d == self.dim
            at += v.shape[0]
        if at != n:
            raise RuntimeError(f"server answered {at} of {n} keys")
        return out, found

    def GetParameter(self, keys, perf: bool = True) -> torch.Tensor:
        k = _keys(keys)
        return self._collect_get(self._issue_get(k, perf), k.numel())[0]

    def GetParameterWithMask(self, keys) -> Tuple[torch.Tensor, torch.Tensor]:
        k = _keys(keys)
        return self._collect_get(self._issue_get(k, True), k.numel())

    def _send_records(self, stub, keys, values) -> int:
        k = _keys(keys)
        v = torch.as_tensor(values, dtype=torch.float32).contiguous()
        assert v.shape == (k.numel(), self.dim)
        futs = [stub.future(PutParameterRequest(parameter_value=pack_records(k[s:s + MAX_PARAMETER_BATCH], v[s:s + MAX_PARAMETER_BATCH])),
                            timeout=self.timeout_s) for s in range(0, k.numel(), MAX_PARAMETER_BATCH)]
        return sum(1 for f in futs if f.result().sucess)

    def PutParameter(self, keys, values) -> bool:
        self._send_records(self._put, keys, values)
        return True

    def UpdateParameter(self, keys, grads) -> int:
        self._send_records(self._upd, keys, grads)
        return int(_keys(keys).numel())

    def _command(self, command: int, arg1=(), arg2=()) -> str:
        return self._cmd(CommandRequest(command=command, arg1=list(arg1), arg2=list(arg2)), timeout=self.timeout_s).reply

    def ClearPS(self) -> bool:
        self._command(CLEAR_PS)
        return True

    def LoadFakeData(self, n: int) -> bool:
        self._command(LOAD_FAKE_DATA, [struct.pack("<q", int(n))])
        return True

    def LoadCkpt(self, model_config_path=None, emb_file_path=None) -> bool:
        files = emb_file_path if isinstance(emb_file_path, (list, tuple)) else [emb_file_path or model_config_path]
        cfg = model_config_path if isinstance(model_config_path, (list, tuple)) else [model_config_path or ""]
        self._command(RELOAD_PS, [str(c).encode() for c in cfg], [str(p).encode() for p in files])
        return True

    def SaveCkpt(self, path: str) -> bool:
        self._command(SAVE_PS, [str(path).encode()])
        return True

    def Stats(self) -> dict:
        a, b, c = (int(x) for x in self._command(STATS).split())
        return {"keys_stored": a, "requests": b, "keys_served": c}

    def HealthCheck(self, service: str = "") -> bool:
        """True when the server reports SERVING for ``service`` through the standard gRPC health protocol."""
        req = (b"\x0a" + bytes([len(service)]) + service.encode()) if service else b""
        rep = self._channel.unary_unary("/grpc.health.v1.Health/Check")(req, timeout=self.timeout_s)
        return rep == b"\x08\x01"

    def Reflect(self, **request) -> "ServerReflectionResponse":
        """One server-reflection exchange, e.g. ``Reflect(list_services="")`` or
        ``Reflect(file_containing_symbol="xmhps.ParameterService")``."""
        call = self._channel.stream_stream(f"/{REFLECTION_SERVICES[0]}/ServerReflectionInfo",
                                           request_serializer=ServerReflectionRequest.SerializeToString,
                                           response_deserializer=ServerReflectionResponse.FromString)
        return next(iter(call(iter([ServerReflectionRequest(**request)]), timeout=self.timeout_s)))

    def ListServices(self) -> List[str]:
        return [s.name for s in self.Reflect(list_services="").list_services_response.service]

    # asynchronous form (src/rdma_ps/base_client.h:6-47) -----------------------------------------
    def InitThread(self, n: int = 1) -> None:
        pass                                                      # gRPC futures need no worker threads

    def GetParameterAsync(self, keys) -> int:
        k = _keys(keys)
        rid = self._next_rpc
        self._next_rpc += 1
        self._rpcs[rid] = [self._issue_get(k, False), k.numel(), None]
        return rid

    def QueryRPCFinished(self, rpc_id: int) -> bool:
        return all(f.done() for f in self._rpcs[rpc_id][0])

    def WaitRPCFinish(self, rpc_id: int) -> None:
        r = self._rpcs[rpc_id]
        if r[2] is None:
            r[2] = self._collect_get(r[0], r[1])[0]

    def GetReceiveBuffer(self, rpc_id: int) -> torch.Tensor:
        self.WaitRPCFinish(rpc_id)
        return self._rpcs[rpc_id][2]

    def RevokeRPCResource(self, rpc_id: int) -> None:
        self._rpcs.pop(rpc_id, None)

    def close(self) -> None:
        if self._channel is not None:
            self._channel.close()
            self._channel = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def serve_shards(servers: List[ParameterServer], host: str = "127.0.0.1") -> List[GrpcParameterServer]:
    """One gRPC endpoint per shard (the reference starts one server process per shard, src/grpc_ps/grpc_ps_server.cpp)."""
    return [GrpcParameterServer(s, 0, host) for s in servers]

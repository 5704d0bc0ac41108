"""The daemon's statistics in the Prometheus text format, for a scraper.

The reference's observability is its log (``src/mccs/src/main.rs:33-65``); this service keeps
counters per communicator and per tenant and hands them out through the ``stats`` admin
command (``csrc/daemon/admin.cc``). This tool turns one answer into exposition text, or serves
it over HTTP:

    python -m mccs_b200.utils.metrics --admin-port 5000 --once        # print and exit
    python -m mccs_b200.utils.metrics --admin-port 5000 --listen 9464 # GET /metrics

Metrics (``comm`` = communicator id, which is also the tenant id of the arbiter):
``mccs_clients``, ``mccs_allocations``, ``mccs_allocated_bytes``;
``mccs_client_allocations{client, pid, app}``, ``mccs_client_allocated_bytes``, ``mccs_client_communicators``
(what each client holds: the quantities the ``[limits]`` table bounds);
``mccs_comm_planned_total``, ``mccs_comm_completed_total`` (kernel launches: a fused launch
counts once), ``mccs_comm_fused_launches_total``, ``mccs_comm_fused_members_total``,
``mccs_comm_config_epoch``, ``mccs_comm_paused``, ``mccs_comm_async_error``,
``mccs_comm_device_error``, ``mccs_comm_info{variant, launch, transport, nranks}``;
``mccs_tenant_admitted_total``, ``mccs_tenant_admitted_bytes_total``,
``mccs_tenant_deferred_total{reason}``, ``mccs_tenant_outstanding_bytes``,
``mccs_tenant_weight``, ``mccs_tenant_priority``.
"""
from __future__ import annotations

import argparse
import sys
from http.server import BaseHTTPRequestHandler, HTTPServer
from typing import Dict, List

from ..client import admin_request


def _esc(value) -> str:
    return str(value).replace("\\", "\\\\").replace('"', '\\"').replace("\n", " ")


def _line(name: str, labels: Dict[str, object], value) -> str:
    lab = ",".join(f'{k}="{_esc(v)}"' for k, v in labels.items())
    return f"{name}{{{lab}}} {value}" if lab else f"{name} {value}"


def render(stats: dict) -> str:
    """Exposition text from the ``stats`` object of the daemon's answer."""
    out: List[str] = []

    def family(name: str, kind: str, help_: str, rows: List[str]) -> None:
        if rows:
            out.append(f"# HELP {name} {help_}")
            out.append(f"# TYPE {name} {kind}")
            out.extend(rows)

    family("mccs_clients", "gauge", "client processes connected to the daemon", [_line("mccs_clients", {}, int(stats.get("clients", 0)))])
    family("mccs_allocations", "gauge", "device allocations handed out", [_line("mccs_allocations", {}, int(stats.get("allocations", 0)))])
    family("mccs_allocated_bytes", "gauge", "bytes of device memory handed out",
           [_line("mccs_allocated_bytes", {}, int(stats.get("allocated_bytes", 0)))])
    holders = stats.get("client_list", [])
    for name, key, help_ in (("mccs_client_allocations", "allocations", "allocations a client holds"),
                             ("mccs_client_allocated_bytes", "allocated_bytes", "bytes of device memory a client holds"),
                             ("mccs_client_communicators", "communicators", "communicator ranks a client holds")):
        family(name, "gauge", help_, [_line(name, {"client": h.get("id", 0), "pid": h.get("pid", 0), "app": h.get("app", "")}, int(h.get(key, 0)))
                                      for h in holders])
    comms = stats.get("communicators", {})
    per_comm = [
        ("mccs_comm_planned_total", "counter", "collectives planned", "planned"),
        ("mccs_comm_completed_total", "counter", "kernel launches completed (a fused launch counts once)", "completed"),
        ("mccs_comm_fused_launches_total", "counter", "launches that carried several AllReduces", "fused_launches"),
        ("mccs_comm_fused_members_total", "counter", "AllReduces carried by fused launches", "fused_members"),
        ("mccs_comm_config_epoch", "gauge", "live reconfigurations applied", "config_epoch"),
        ("mccs_comm_paused", "gauge", "1 while the communicator is paused", "paused"),
        ("mccs_comm_async_error", "gauge", "first error of the communicator (0 = none)", "async_error"),
        ("mccs_comm_device_error", "gauge", "error reported by a kernel (0 = none)", "device_error"),
    ]
    for name, kind, help_, key in per_comm:
        family(name, kind, help_, [_line(name, {"comm": cid}, int(c.get(key, 0))) for cid, c in sorted(comms.items())])
    family("mccs_comm_info", "gauge", "what the communicator last ran and how it is served",
           [_line("mccs_comm_info", {"comm": cid, "variant": c.get("last_variant", ""), "launch": "client" if c.get("client_launch") else "daemon",
                                     "transport": c.get("transport", ""), "nranks": c.get("nranks", 0)}, 1)
            for cid, c in sorted(comms.items())])
    tenants = stats.get("qos", {}).get("tenants", {})
    family("mccs_tenant_admitted_total", "counter", "collectives (or slices) admitted by the arbiter",
           [_line("mccs_tenant_admitted_total", {"comm": t}, int(v.get("admitted", 0))) for t, v in sorted(tenants.items())])
    family("mccs_tenant_admitted_bytes_total", "counter", "bytes admitted by the arbiter",
           [_line("mccs_tenant_admitted_bytes_total", {"comm": t}, int(v.get("bytes_admitted", 0))) for t, v in sorted(tenants.items())])
    family("mccs_tenant_deferred_total", "counter", "times a request was told to wait, by reason",
           [_line("mccs_tenant_deferred_total", {"comm": t, "reason": r}, int(v.get("deferred_" + r, 0)))
            for t, v in sorted(tenants.items()) for r in ("window", "backlog", "fairness", "residency")])
    family("mccs_tenant_outstanding_bytes", "gauge", "bytes admitted and not yet completed",
           [_line("mccs_tenant_outstanding_bytes", {"comm": t}, int(v.get("outstanding_bytes", 0))) for t, v in sorted(tenants.items())])
    family("mccs_tenant_weight", "gauge", "share of the tenant under contention",
           [_line("mccs_tenant_weight", {"comm": t}, float(v.get("weight", 1))) for t, v in sorted(tenants.items())])
    family("mccs_tenant_priority", "gauge", "1 = high-priority stream", [_line("mccs_tenant_priority", {"comm": t}, int(v.get("priority", 0)))
                                                                       for t, v in sorted(tenants.items())])
    return "\n".join(out) + "\n"


def scrape(admin_port: int, host: str = "127.0.0.1") -> str:
    rep = admin_request(admin_port, {"cmd": "stats"}, host=host)
    if rep.get("status") != "ok":
        raise RuntimeError(f"the daemon answered {rep}")
    return render(rep["stats"])


def serve(admin_port: int, listen: int, host: str = "127.0.0.1", bind: str = "127.0.0.1") -> HTTPServer:
    """An HTTP server whose ``/metrics`` asks the daemon at every request. Returns the server
    (``serve_forever()`` runs it, ``server_address[1]`` is the port when ``listen`` was 0)."""

    class Handler(BaseHTTPRequestHandler):
        def do_GET(self):  # noqa: N802
            if self.path.split("?")[0] != "/metrics":
                self.send_error(404)
                return
            try:
                body = scrape(admin_port, host).encode()
            except Exception as e:  # the daemon is gone or does not answer: say so to the scraper
                self.send_error(503, str(e))
                return
            self.send_response(200)
            self.send_header("Content-Type", "text/plain; version=0.0.4; charset=utf-8")
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

        def log_message(self, *args):
            pass

    return HTTPServer((bind, listen), Handler)


def main() -> int:
    ap = argparse.ArgumentParser(description="Prometheus text exposition of the daemon's statistics")
    ap.add_argument("--admin-port", type=int, required=True, help="the daemon's admin port (listen_port of its configuration)")
    ap.add_argument("--admin-host", default="127.0.0.1")
    ap.add_argument("--once", action="store_true", help="print the metrics once and exit")
    ap.add_argument("--listen", type=int, default=9464, help="port of the /metrics endpoint")
    ap.add_argument("--bind", default="127.0.0.1")
    a = ap.parse_args()
    if a.once:
        sys.stdout.write(scrape(a.admin_port, a.admin_host))
        return 0
    srv = serve(a.admin_port, a.listen, a.admin_host, a.bind)
    print(f"serving http://{a.bind}:{srv.server_address[1]}/metrics", flush=True)
    try:
        srv.serve_forever()
    except KeyboardInterrupt:
        pass
    return 0


if __name__ == "__main__":
    sys.exit(main())

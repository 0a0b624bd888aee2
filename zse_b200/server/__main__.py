"""``python -m zse_b200.server --model model.zse --port 8000`` (zse-engine/zse_engine/server/__main__.py:24-84)."""
import argparse
import asyncio

from .app import ZSEServer


def main(argv=None):
    ap = argparse.ArgumentParser(prog="zse_b200.server")
    ap.add_argument("--model", default=None, help=".zse model file (omit for mock mode)")
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--admin-key", default=None)
    ap.add_argument("--db-path", default="~/.zse/server.db")
    ap.add_argument("--model-name", default="zse-model")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--require-auth", action="store_true")
    ap.add_argument("-q", "--quiet", action="store_true")
    a = ap.parse_args(argv)
    srv = ZSEServer(a.model, a.host, a.port, a.admin_key, a.db_path, a.model_name, a.quiet, a.tp,
                    require_auth=a.require_auth)
    try:
        asyncio.run(srv.run_forever())
    except KeyboardInterrupt:
        srv.close()


if __name__ == "__main__":
    main()

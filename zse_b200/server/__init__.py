from .app import ZSEServer
from .auth import AuthManager, AuthResult
from .database import ServerDatabase
from .router import Request, Response, Router

__all__ = ["ZSEServer", "AuthManager", "AuthResult", "ServerDatabase", "Request", "Response", "Router"]

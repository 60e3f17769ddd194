from .auth import AuthManager
from .input_validator import InputValidator
from .rate_limiter import RateLimiter, SecureConversationalChat

"""Process-wide logger.

Format: ``[time host:pid][file:line][LEVEL] message`` as in the reference
(msamp/common/utils/logging.py:20-87).  Colours are ANSI escapes emitted only when the stream is a
terminal, so no third-party colour package is needed.
"""
import logging
import os
import socket
import sys


class _Formatter(logging.Formatter):
    _COLOURS = {'DEBUG': '\033[37m', 'INFO': '\033[0m', 'WARNING': '\033[33m', 'ERROR': '\033[31m', 'CRITICAL': '\033[1;31m'}

    def __init__(self, colour):
        host = socket.gethostname()
        super().__init__(
            f'[%(asctime)s {host}:{os.getpid()}][%(filename)s:%(lineno)s][%(levelname)s] %(message)s',
            datefmt='%Y-%m-%d %H:%M:%S'
        )
        self._colour = colour

    def format(self, record):
        text = super().format(record)
        if self._colour:
            return f'{self._COLOURS.get(record.levelname, "")}{text}\033[0m'
        return text


class MsAmpLogger(logging.Logger):
    """Logger with a ``log_and_raise`` helper."""
    def __init__(self, name, level=logging.INFO):
        super().__init__(name, level)
        handler = logging.StreamHandler(sys.stdout)
        handler.setFormatter(_Formatter(colour=sys.stdout.isatty()))
        self.addHandler(handler)
        self.propagate = False

    def log_and_raise(self, exception, msg, *args):
        """Log ``msg`` at error level and raise ``exception(msg)``."""
        text = msg % args if args else msg
        self.error(text, stacklevel=2)
        raise exception(text)


logger = MsAmpLogger('msamp', level=getattr(logging, os.environ.get('MSAMP_LOG_LEVEL', 'INFO').upper(), logging.INFO))

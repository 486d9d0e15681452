import os
import sys

from .app import main

try:
    code = main()
    sys.stdout.flush()
except BrokenPipeError:
    # the reader of our output went away (`... | head`): not an error; keep the interpreter from complaining at exit
    os.dup2(os.open(os.devnull, os.O_WRONLY), sys.stdout.fileno())
    code = 0
sys.exit(code)

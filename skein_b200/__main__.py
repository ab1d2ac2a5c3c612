"""`python -m skein_b200 <sub-command>` is the `skein` command."""
import sys

from .cli.main import main

sys.exit(main())

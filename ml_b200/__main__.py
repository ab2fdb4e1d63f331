import sys

from .gpt import main

sys.exit(main())

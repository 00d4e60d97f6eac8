"""``python -m minisgl --model <path> ...`` starts the server (python/minisgl/__main__.py of the reference)."""
from minisgl.server.launch import launch_server


def main() -> None:
    launch_server()


if __name__ == "__main__":
    main()
